// Host-side argument checking and geometry resolution for every operator.
//
// These functions reproduce the checks, defaults and error codes of the reference's
// TensorMath functions (paths below are into the Z-Ant tree) so that a caller swapping
// back ends sees the same accept/reject behaviour.  They run before anything touches the
// device and are usable without a GPU.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#include "status.hpp"

namespace zb {

inline bool bytes_eq(const char* s, size_t len, const char* lit) {
    return s != nullptr && std::strlen(lit) == len && std::memcmp(s, lit, len) == 0;
}

inline size_t numel(const size_t* s, size_t r) {
    size_t n = 1;
    for (size_t i = 0; i < r; ++i) n *= s[i];
    return n;
}

inline size_t dtype_size(int32_t dt) { return (dt == ZANT_F32 || dt == ZANT_I32) ? 4 : 1; }
inline bool dtype_valid(int32_t dt) { return dt >= ZANT_F32 && dt <= ZANT_I32; }

// ONNX gives a zero point the type of its tensor.  The fast quantized kernels rely on it: they fill
// padded pixels with the zero point as a byte, so a value outside the type's range would make them
// disagree with the generic kernel.  Such a value is refused everywhere instead.
inline int32_t check_zero_point(int32_t dtype, int32_t zp, const char* what) {
    const int lo = dtype == ZANT_U8 ? 0 : -128, hi = dtype == ZANT_U8 ? 255 : 127;
    if ((dtype == ZANT_I8 || dtype == ZANT_U8) && (zp < lo || zp > hi))
        return fail(ZANT_E_INVALID_INPUT, "%s zero point %d is outside [%d, %d]", what, zp, lo, hi);
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ conv
// Everything a convolution kernel needs; produced by both the reference-rule resolver (f32
// Conv) and the ONNX-rule resolver (QLinearConv).
struct ConvGeom {
    int N, C, H, W;        // input
    int M, Cg, KH, KW;     // filters, channels per group
    int sh, sw, dh, dw;
    int pt, pl, pb, pr;
    int OH, OW;
    int G;                 // groups
};

inline bool fits_int(size_t v) { return v <= (size_t)std::numeric_limits<int>::max(); }

struct StrideDil { size_t sh, sw, dh, dw; };

// Defaults of op_convolution.zig:68-71: one stride/dilation value applies to both axes.
inline StrideDil stride_dil_defaults(const size_t* stride, size_t ns, const size_t* dil, size_t nd) {
    StrideDil r;
    r.sh = ns > 0 ? stride[0] : 1;
    r.sw = ns > 1 ? stride[1] : r.sh;
    r.dh = (dil && nd > 0) ? dil[0] : 1;
    r.dw = (dil && nd > 1) ? dil[1] : r.dh;
    return r;
}

// SAME_UPPER / SAME_LOWER split (op_convolution.zig:90-110).  Returns false when the total
// would be negative (the reference computes it in usize, where that wraps).
inline bool same_pads(size_t in, size_t stride, size_t dil_k, bool upper, size_t& begin, size_t& end) {
    const size_t out = (in + stride - 1) / stride;
    const long long total = (long long)((out - 1) * stride + dil_k) - (long long)in;
    if (total < 0) return false;
    const size_t t = (size_t)total;
    if (upper) { begin = t / 2; end = t - begin; }
    else       { end = t / 2; begin = t - end; }
    return true;
}

inline int32_t fill_geom(ConvGeom& g, const size_t* xs, const size_t* ws, const StrideDil& sd,
                         size_t pt, size_t pl, size_t pb, size_t pr, size_t groups) {
    const size_t dkh = (ws[2] - 1) * sd.dh + 1, dkw = (ws[3] - 1) * sd.dw + 1;
    const size_t PH = xs[2] + pt + pb, PW = xs[3] + pl + pr;
    if (PH < dkh || PW < dkw) return fail(ZANT_E_INVALID_DIMENSIONS, "kernel larger than padded input");
    const size_t OH = (PH - dkh) / sd.sh + 1, OW = (PW - dkw) / sd.sw + 1;
    const size_t all[] = {xs[0], xs[1], xs[2], xs[3], ws[0], ws[1], ws[2], ws[3], sd.sh, sd.sw, sd.dh, sd.dw,
                          pt, pl, pb, pr, OH, OW, PH, PW};
    for (size_t v : all) if (!fits_int(v)) return fail(ZANT_E_TOO_LARGE, "dimension exceeds int range");
    g.N = (int)xs[0]; g.C = (int)xs[1]; g.H = (int)xs[2]; g.W = (int)xs[3];
    g.M = (int)ws[0]; g.Cg = (int)ws[1]; g.KH = (int)ws[2]; g.KW = (int)ws[3];
    g.sh = (int)sd.sh; g.sw = (int)sd.sw; g.dh = (int)sd.dh; g.dw = (int)sd.dw;
    g.pt = (int)pt; g.pl = (int)pl; g.pb = (int)pb; g.pr = (int)pr;
    g.OH = (int)OH; g.OW = (int)OW; g.G = (int)groups;
    return ZANT_OK;
}

// OnnxConvLean's argument handling (op_convolution.zig:44-129, :212-217).
inline int32_t conv_resolve_ref(const size_t* xs, size_t xr, const size_t* ws, size_t wr,
                                const size_t* ys, size_t yr,
                                const size_t* stride, size_t ns, const size_t* pads, size_t np,
                                const size_t* dil, size_t nd, size_t group,
                                const char* auto_pad, size_t apl, ConvGeom& g) {
    if (xr != 4 || wr != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "Conv needs 4-D input and kernel");
    if (group != 0 && group != 1) return fail(ZANT_E_INVALID_DIMENSIONS, "Conv supports group 1 only (got %zu)", group);
    const StrideDil sd = stride_dil_defaults(stride, ns, dil, nd);
    if (sd.sh == 0 || sd.sw == 0 || sd.dh == 0 || sd.dw == 0 || ws[2] == 0 || ws[3] == 0)
        return fail(ZANT_E_INVALID_DIMENSIONS, "zero stride, dilation or kernel extent");
    size_t pt = 0, pl = 0, pb = 0, pr = 0;
    if (auto_pad) {  // pads are only looked at inside this branch, as in the reference
        const bool up = bytes_eq(auto_pad, apl, "SAME_UPPER"), lo = bytes_eq(auto_pad, apl, "SAME_LOWER");
        if (up || lo) {
            if (!same_pads(xs[2], sd.sh, (ws[2] - 1) * sd.dh + 1, up, pt, pb) ||
                !same_pads(xs[3], sd.sw, (ws[3] - 1) * sd.dw + 1, up, pl, pr))
                return fail(ZANT_E_INVALID_PADDING, "SAME padding would be negative");
        } else if (bytes_eq(auto_pad, apl, "NOTSET")) {
            if (!pads) return fail(ZANT_E_INVALID_PADDING, "auto_pad NOTSET without pads");
            if (np >= 4) { pt = pads[0]; pl = pads[1]; pb = pads[2]; pr = pads[3]; }
        }
        // "VALID" and unknown strings: no padding
    }
    int32_t st = fill_geom(g, xs, ws, sd, pt, pl, pb, pr, 1);
    if (st != ZANT_OK) return st;
    if (ws[1] != xs[1]) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "kernel channels %zu != input channels %zu", ws[1], xs[1]);
    if (yr != 4 || (int)ys[0] != g.N || (int)ys[1] != g.M || (int)ys[2] != g.OH || (int)ys[3] != g.OW)
        return fail(ZANT_E_INVALID_DIMENSIONS, "output shape does not match [%d,%d,%d,%d]", g.N, g.M, g.OH, g.OW);
    return ZANT_OK;
}

// Output shape computed by the allocating wrapper OnnxConv (op_convolution.zig:682-732).
inline int32_t conv_output_shape_ref(const size_t* xs, size_t xr, const size_t* ws, size_t wr,
                                     const size_t* stride, size_t ns, const size_t* pads, size_t np,
                                     const size_t* dil, size_t nd, const char* auto_pad, size_t apl,
                                     size_t out[4]) {
    if (xr != 4 || wr != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "Conv needs 4-D input and kernel");
    const StrideDil sd = stride_dil_defaults(stride, ns, dil, nd);
    if (sd.sh == 0 || sd.sw == 0 || ws[2] == 0 || ws[3] == 0) return fail(ZANT_E_INVALID_DIMENSIONS, "zero stride or kernel");
    const size_t dkh = (ws[2] - 1) * sd.dh + 1, dkw = (ws[3] - 1) * sd.dw + 1;
    size_t ph = 0, pw = 0;
    bool same = false;
    if (auto_pad) {
        if (bytes_eq(auto_pad, apl, "VALID")) {
        } else if (bytes_eq(auto_pad, apl, "SAME_UPPER") || bytes_eq(auto_pad, apl, "SAME_LOWER")) {
            same = true;
        } else if (bytes_eq(auto_pad, apl, "NOTSET")) {
            if (pads) {
                if (np < 4) return fail(ZANT_E_INVALID_PADDING, "pads needs 4 entries");
                ph = pads[0] + pads[2]; pw = pads[1] + pads[3];
            }
        } else {
            return fail(ZANT_E_INVALID_PADDING, "unknown auto_pad");
        }
    } else if (pads && np >= 4) {
        ph = pads[0] + pads[2]; pw = pads[1] + pads[3];
    }
    out[0] = xs[0]; out[1] = ws[0];
    if (same) {
        out[2] = (xs[2] + sd.sh - 1) / sd.sh; out[3] = (xs[3] + sd.sw - 1) / sd.sw;
    } else {
        if (xs[2] + ph < dkh || xs[3] + pw < dkw) return fail(ZANT_E_INVALID_DIMENSIONS, "kernel larger than input");
        out[2] = (xs[2] + ph - dkh) / sd.sh + 1; out[3] = (xs[3] + pw - dkw) / sd.sw + 1;
    }
    return ZANT_OK;
}

// ONNX rules for QLinearConv: explicit pads unless auto_pad asks otherwise; groups allowed.
inline int32_t conv_resolve_onnx(const size_t* xs, size_t xr, const size_t* ws, size_t wr,
                                 const size_t* ys, size_t yr,
                                 const size_t* stride, size_t ns, const size_t* pads, size_t np,
                                 const size_t* dil, size_t nd, size_t group, int32_t auto_pad, ConvGeom& g) {
    if (xr != 4 || wr != 4 || yr != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "QLinearConv needs 4-D tensors");
    const size_t G = group == 0 ? 1 : group;
    if (xs[1] % G != 0 || ws[0] % G != 0 || ws[1] != xs[1] / G)
        return fail(ZANT_E_INVALID_DIMENSIONS, "channels / filters not divisible by group %zu", G);
    const StrideDil sd = stride_dil_defaults(stride, ns, dil, nd);
    if (sd.sh == 0 || sd.sw == 0 || sd.dh == 0 || sd.dw == 0 || ws[2] == 0 || ws[3] == 0)
        return fail(ZANT_E_INVALID_DIMENSIONS, "zero stride, dilation or kernel extent");
    size_t pt = 0, pl = 0, pb = 0, pr = 0;
    if (auto_pad == ZANT_PAD_NOTSET) {
        if (pads && np >= 4) { pt = pads[0]; pl = pads[1]; pb = pads[2]; pr = pads[3]; }
    } else if (auto_pad == ZANT_PAD_SAME_UPPER || auto_pad == ZANT_PAD_SAME_LOWER) {
        const bool up = auto_pad == ZANT_PAD_SAME_UPPER;
        // ONNX clamps a negative total to zero.
        if (!same_pads(xs[2], sd.sh, (ws[2] - 1) * sd.dh + 1, up, pt, pb)) { pt = pb = 0; }
        if (!same_pads(xs[3], sd.sw, (ws[3] - 1) * sd.dw + 1, up, pl, pr)) { pl = pr = 0; }
    } else if (auto_pad != ZANT_PAD_VALID) {
        return fail(ZANT_E_INVALID_PADDING, "unknown auto_pad %d", auto_pad);
    }
    int32_t st = fill_geom(g, xs, ws, sd, pt, pl, pb, pr, G);
    if (st != ZANT_OK) return st;
    if ((int)ys[0] != g.N || (int)ys[1] != g.M || (int)ys[2] != g.OH || (int)ys[3] != g.OW)
        return fail(ZANT_E_INVALID_DIMENSIONS, "output shape does not match [%d,%d,%d,%d]", g.N, g.M, g.OH, g.OW);
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ pooling
struct PoolGeom {
    int NC, H, W, OH, OW, KH, KW, sh, sw, dh, dw, pt, pl;
};

// get_pooling_output_shape, op_pooling.zig:16-35.
inline int32_t pooling_output_shape(const size_t* xs, size_t xr, const size_t k[2], const size_t s[2], size_t out[4]) {
    if (xr != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "pooling needs a 4-D input");
    if (k[0] == 0 || k[1] == 0 || s[0] == 0 || s[1] == 0) return fail(ZANT_E_WRONG_STRIDE, "zero kernel or stride");
    if (k[0] > xs[2] || k[1] > xs[3]) return fail(ZANT_E_INVALID_DIMENSIONS, "kernel larger than input");
    out[0] = xs[0]; out[1] = xs[1];
    out[2] = (xs[2] - k[0]) / s[0] + 1;
    out[3] = (xs[3] - k[1]) / s[1] + 1;
    return ZANT_OK;
}

// get_onnx_maxpool_output_shape, op_pooling.zig:477-567.
inline int32_t maxpool_output_shape(const size_t* xs, size_t xr, const size_t* k, const size_t* s,
                                    const size_t* d, const size_t* pads, int32_t auto_pad, int32_t ceil_mode,
                                    size_t out[4]) {
    if (xr != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "MaxPool needs a 4-D input");
    if (!k || !s || !d) return fail(ZANT_E_NULL_POINTER, "kernel_shape/strides/dilations");
    if (k[0] == 0 || k[1] == 0 || s[0] == 0 || s[1] == 0) return fail(ZANT_E_WRONG_STRIDE, "zero kernel or stride");
    const size_t ekh = (k[0] - 1) * d[0] + 1, ekw = (k[1] - 1) * d[1] + 1;
    long long ph = 0, pw = 0;
    switch (auto_pad) {
        case ZANT_PAD_NOTSET:
            if (!pads) return fail(ZANT_E_NULL_POINTER, "pads");
            ph = (long long)(pads[0] + pads[2]); pw = (long long)(pads[1] + pads[3]);
            break;
        case ZANT_PAD_VALID: break;
        case ZANT_PAD_SAME_UPPER:
        case ZANT_PAD_SAME_LOWER: {
            const size_t oh = (xs[2] + s[0] - 1) / s[0], ow = (xs[3] + s[1] - 1) / s[1];
            ph = (long long)((oh - 1) * s[0] + ekh) - (long long)xs[2];
            pw = (long long)((ow - 1) * s[1] + ekw) - (long long)xs[3];
            if (ph < 0 || pw < 0) return fail(ZANT_E_INVALID_PADDING, "SAME padding would be negative");
            break;
        }
        default: return fail(ZANT_E_INVALID_PADDING, "unknown auto_pad %d", auto_pad);
    }
    const long long nh = (long long)xs[2] + ph - (long long)ekh, nw = (long long)xs[3] + pw - (long long)ekw;
    if (nh < 0 || nw < 0) return fail(ZANT_E_INVALID_DIMENSIONS, "kernel larger than padded input");
    out[0] = xs[0]; out[1] = xs[1];
    if (ceil_mode) {
        out[2] = ((size_t)nh + s[0] - 1) / s[0] + 1; out[3] = ((size_t)nw + s[1] - 1) / s[1] + 1;
    } else {
        out[2] = (size_t)nh / s[0] + 1; out[3] = (size_t)nw / s[1] + 1;
    }
    return ZANT_OK;
}

// Pad resolution of lean_onnx_maxpool (op_pooling.zig:587-618): SAME_* is derived from the
// OUTPUT shape and the undilated kernel.
inline int32_t pool_resolve(const size_t* xs, size_t xr, const size_t* ys, size_t yr,
                            const size_t* k, size_t nk, const size_t* s, size_t nst,
                            const size_t* d, size_t nd, const size_t* pads, size_t np,
                            int32_t auto_pad, PoolGeom& g) {
    if (xr != 4 || yr != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "MaxPool needs 4-D tensors");
    if (!k || !s || !d || nk < 2 || nst < 2 || nd < 2) return fail(ZANT_E_INVALID_DIMENSIONS, "kernel_shape/strides/dilations need 2 entries");
    if (ys[0] != xs[0] || ys[1] != xs[1]) return fail(ZANT_E_INVALID_DIMENSIONS, "batch/channels differ between input and output");
    size_t pt = 0, pl = 0;
    switch (auto_pad) {
        case ZANT_PAD_NOTSET:
            if (pads && np >= 4) { pt = pads[0]; pl = pads[1]; }
            break;
        case ZANT_PAD_VALID: break;
        case ZANT_PAD_SAME_UPPER:
        case ZANT_PAD_SAME_LOWER: {
            const long long th = (long long)((ys[2] - 1) * s[0] + k[0]) - (long long)xs[2];
            const long long tw = (long long)((ys[3] - 1) * s[1] + k[1]) - (long long)xs[3];
            if (th < 0 || tw < 0) return fail(ZANT_E_INVALID_PADDING, "SAME padding would be negative");
            if (auto_pad == ZANT_PAD_SAME_UPPER) { pt = (size_t)th / 2; pl = (size_t)tw / 2; }
            else { pt = (size_t)th - (size_t)th / 2; pl = (size_t)tw - (size_t)tw / 2; }
            break;
        }
        default: return fail(ZANT_E_INVALID_PADDING, "unknown auto_pad %d", auto_pad);
    }
    const size_t all[] = {xs[0] * xs[1], xs[2], xs[3], ys[2], ys[3], k[0], k[1], s[0], s[1], d[0], d[1], pt, pl};
    for (size_t v : all) if (!fits_int(v)) return fail(ZANT_E_TOO_LARGE, "dimension exceeds int range");
    g.NC = (int)(xs[0] * xs[1]); g.H = (int)xs[2]; g.W = (int)xs[3]; g.OH = (int)ys[2]; g.OW = (int)ys[3];
    g.KH = (int)k[0]; g.KW = (int)k[1]; g.sh = (int)s[0]; g.sw = (int)s[1]; g.dh = (int)d[0]; g.dw = (int)d[1];
    g.pt = (int)pt; g.pl = (int)pl;
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ matmul / gemm
struct MatGeom { size_t M, N, K; };

// mat_mul, op_mat_mul.zig:22-57.
inline int32_t matmul_check(const size_t* as, size_t ar, const size_t* bs, size_t br,
                            const size_t* ys, size_t yr, MatGeom& g) {
    if (ar != br) return fail(ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE, "ranks differ (%zu vs %zu)", ar, br);
    if (ar < 2) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "MatMul needs rank >= 2");
    if (as[ar - 1] != bs[ar - 2]) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "A cols %zu != B rows %zu", as[ar - 1], bs[ar - 2]);
    g.M = as[ar - 2]; g.N = bs[ar - 1]; g.K = as[ar - 1];
    if (g.M * g.N == 0 || g.K == 0) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "empty operand");
    if (yr < 2 || ys[yr - 2] != g.M || ys[yr - 1] != g.N) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output is not [%zu,%zu]", g.M, g.N);
    return ZANT_OK;
}

struct GemmGeom {
    size_t rows, cols, K;
    size_t batch;          // A.shape[0]*A.shape[1]; the alpha/beta passes cover all of it
    int c_mode;            // 0 none, 1 same size, 2 broadcast
    size_t c_rows, c_cols; // C's last two dims (broadcast mode)
    size_t c_ch;           // C.shape[1]
};

// gemm, op_gemm.zig:15-61.
inline int32_t gemm_check(const size_t* as, size_t ar, const size_t* bs, size_t br,
                          const size_t* cs, size_t cr, bool has_c, bool ta, bool tb, float beta,
                          const size_t* ys, size_t yr, GemmGeom& g) {
    if (ar != 4 || br != 4) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "Gemm operands must be 4-D");
    if (as[0] != bs[0] || as[1] != bs[1]) return fail(ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE, "batch/channel dims differ");
    const size_t condA = ta ? as[2] : as[3], condB = tb ? bs[3] : bs[2];
    g.rows = ta ? as[3] : as[2];
    g.cols = tb ? bs[2] : bs[3];
    if (condA != condB) return fail(ZANT_E_INPUT_TENSOR_DIMENSION_MISMATCH, "inner dims %zu vs %zu", condA, condB);
    g.K = condA;
    g.batch = as[0] * as[1];
    g.c_mode = 0; g.c_rows = g.c_cols = g.c_ch = 1;
    if (has_c) {
        if (cr != 4) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "C must be 4-D");
        if (cs[0] != as[0] || cs[1] != as[1]) return fail(ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE, "C batch/channel dims differ");
        if ((cs[2] != g.rows && cs[2] != 1) || (cs[3] != g.cols && cs[3] != 1))
            return fail(ZANT_E_INCOMPATIBLE_BROADCAST_SHAPES, "C [%zu,%zu] does not broadcast to [%zu,%zu]", cs[2], cs[3], g.rows, g.cols);
        if (beta != 0.0f) {
            g.c_mode = (numel(cs, 4) == g.batch * g.rows * g.cols) ? 1 : 2;
            g.c_rows = cs[2]; g.c_cols = cs[3]; g.c_ch = cs[1];
        }
    }
    if (yr != 4 || ys[0] != as[0] || ys[1] != as[1] || ys[2] != g.rows || ys[3] != g.cols)
        return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output is not [..,%zu,%zu]", g.rows, g.cols);
    if (g.rows * g.cols == 0 || g.K == 0) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "empty operand");
    return ZANT_OK;
}

// gemm_lean as generated code calls it (src/codeGen/hardcoded/hardcoded_sentiment_it.zig:137): lean_gemm itself
// has no rank check, multiplies the last two dimensions (op_gemm.zig:128, op_mat_mul.zig:92-172) and reads C's
// last two (one) dimensions for the broadcast (op_gemm.zig:150-156).  Operands of rank 1..3 are therefore taken
// as [1,..,1,rows,cols]; for rank-4 operands the rules are those of gemm_check.
inline int32_t gemm_check_lean(const size_t* as, size_t ar, const size_t* bs, size_t br,
                               const size_t* cs, size_t cr, bool has_c, bool ta, bool tb, float beta,
                               const size_t* ys, size_t yr, GemmGeom& g) {
    if (ar < 2 || ar > 4 || br < 2 || br > 4 || yr < 2 || yr > 4 || (has_c && (cr < 1 || cr > 4)))
        return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "Gemm operands must have rank 2..4 (C: 1..4)");
    auto promote = [](const size_t* sh, size_t r, size_t out[4]) {
        for (size_t i = 0; i < 4; ++i) out[i] = i + r < 4 ? 1 : sh[i + r - 4];
    };
    size_t a4[4], b4[4], c4[4] = {1, 1, 1, 1}, y4[4];
    promote(as, ar, a4); promote(bs, br, b4); promote(ys, yr, y4);
    if (has_c) promote(cs, cr, c4);
    return gemm_check(a4, 4, b4, 4, has_c ? c4 : nullptr, has_c ? 4 : 0, has_c, ta, tb, beta, y4, 4, g);
}

// ------------------------------------------------------------------------------------ Add broadcast
struct BcastGeom {
    int rank;
    size_t out_shape[4];
    size_t a_stride[4], b_stride[4];  // element strides of each operand, 0 on broadcast dims
    size_t total;
    bool same_size;
};

// lean_sum_tensors, lib_elementWise_math.zig:70-210.  Equal element counts add index by
// index whatever the shapes; otherwise NumPy right-aligned broadcasting up to rank 4.  (The
// reference derives operand strides from the output shape, which over-runs an operand shaped
// like [C,1,1]; this back end uses each operand's own strides, i.e. the ONNX Add result.)
inline int32_t bcast_resolve(const size_t* as, size_t ar, const size_t* bs, size_t br,
                             const size_t* ys, size_t yr, BcastGeom& g) {
    const size_t an = numel(as, ar), bn = numel(bs, br);
    g.same_size = (an == bn);
    if (g.same_size) {
        g.total = an;
        if (numel(ys, yr) != an) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output holds %zu elements, inputs %zu", numel(ys, yr), an);
        return ZANT_OK;
    }
    const size_t mr = std::max(ar, br);
    if (mr > 4) return fail(ZANT_E_UNSUPPORTED, "broadcast Add above rank 4");
    size_t s1[4] = {1, 1, 1, 1}, s2[4] = {1, 1, 1, 1};
    for (size_t i = 0; i < ar; ++i) s1[mr - ar + i] = as[i];
    for (size_t i = 0; i < br; ++i) s2[mr - br + i] = bs[i];
    g.rank = (int)mr;
    g.total = 1;
    for (size_t d = 0; d < mr; ++d) {
        if (s1[d] != s2[d] && s1[d] != 1 && s2[d] != 1)
            return fail(ZANT_E_INCOMPATIBLE_BROADCAST_SHAPES, "dim %zu: %zu vs %zu", d, s1[d], s2[d]);
        g.out_shape[d] = std::max(s1[d], s2[d]);
        g.total *= g.out_shape[d];
    }
    if (yr != mr) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output rank %zu != %zu", yr, mr);
    for (size_t d = 0; d < mr; ++d)
        if (ys[d] != g.out_shape[d]) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output dim %zu is %zu, expected %zu", d, ys[d], g.out_shape[d]);
    size_t t1 = 1, t2 = 1;
    for (size_t d = mr; d-- > 0;) {
        g.a_stride[d] = s1[d] > 1 ? t1 : 0;
        g.b_stride[d] = s2[d] > 1 ? t2 : 0;
        t1 *= s1[d]; t2 *= s2[d];
    }
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ concat
struct ConcatGeom {
    size_t rank, axis, num_slices, slice;   // slice = elements after the axis
    std::vector<size_t> axis_dim;           // per tensor
    size_t out_axis_dim;
};

// Rank promotion + validation of concatenate / lean_concatenate (lib_shape_math.zig:307-445,
// :463-543).  `out_shape` (max-rank entries) is filled.
inline int32_t concat_resolve(const size_t* const* shapes, const size_t* ranks, size_t nt, int64_t axis,
                              size_t* out_shape, ConcatGeom& g) {
    if (nt == 0) return fail(ZANT_E_EMPTY_TENSOR_LIST, "no tensors to concatenate");
    size_t mr = ranks[0];
    for (size_t t = 0; t < nt; ++t) mr = std::max(mr, ranks[t]);
    if (mr == 0 || mr > 8) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "rank %zu", mr);
    int64_t ax = axis < 0 ? axis + (int64_t)mr : axis;
    if (ax < 0 || ax >= (int64_t)mr) return fail(ZANT_E_AXIS_OUT_OF_BOUNDS, "axis %lld for rank %zu", (long long)axis, mr);
    std::vector<std::vector<size_t>> sh(nt, std::vector<size_t>(mr, 1));
    for (size_t t = 0; t < nt; ++t)
        for (size_t d = 0; d < ranks[t]; ++d) sh[t][mr - ranks[t] + d] = shapes[t][d];
    g.rank = mr; g.axis = (size_t)ax; g.axis_dim.resize(nt); g.out_axis_dim = 0;
    for (size_t t = 0; t < nt; ++t) {
        for (size_t d = 0; d < mr; ++d)
            if (d != g.axis && sh[t][d] != sh[0][d]) return fail(ZANT_E_MISMATCHED_SHAPE, "tensor %zu dim %zu: %zu vs %zu", t, d, sh[t][d], sh[0][d]);
        g.axis_dim[t] = sh[t][g.axis];
        g.out_axis_dim += sh[t][g.axis];
    }
    g.num_slices = 1; g.slice = 1;
    for (size_t d = 0; d < mr; ++d) {
        out_shape[d] = d == g.axis ? g.out_axis_dim : sh[0][d];
        if (d < g.axis) g.num_slices *= sh[0][d];
        if (d > g.axis) g.slice *= sh[0][d];
    }
    return ZANT_OK;
}

// get_concatenate_output_shape, lib_shape_math.zig:582-629.
inline int32_t concat_output_shape_strict(const size_t* const* shapes, const size_t* ranks, size_t nt,
                                          int64_t axis, size_t* out) {
    if (nt == 0) return fail(ZANT_E_EMPTY_TENSOR_LIST, "no tensors to concatenate");
    const size_t rank = ranks[0];
    int64_t ax = axis < 0 ? axis + (int64_t)rank : axis;
    if (ax < 0 || ax >= (int64_t)rank) return fail(ZANT_E_AXIS_OUT_OF_BOUNDS, "axis %lld for rank %zu", (long long)axis, rank);
    for (size_t t = 0; t < nt; ++t) {
        if (ranks[t] != rank) return fail(ZANT_E_MISMATCHED_RANK, "tensor %zu has rank %zu, expected %zu", t, ranks[t], rank);
        for (size_t d = 0; d < rank; ++d)
            if (d != (size_t)ax && shapes[t][d] != shapes[0][d]) return fail(ZANT_E_MISMATCHED_SHAPE, "tensor %zu dim %zu", t, d);
    }
    for (size_t d = 0; d < rank; ++d) {
        out[d] = shapes[0][d];
        if (d == (size_t)ax) { out[d] = 0; for (size_t t = 0; t < nt; ++t) out[d] += shapes[t][d]; }
    }
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ resize
// get_resize_output_shape, lib_shape_math.zig:78-104.
inline int32_t resize_output_shape(const size_t* xs, size_t r, const float* scales, size_t nsc,
                                   const size_t* sizes, size_t nsz, size_t* out) {
    if (!scales && !sizes) return fail(ZANT_E_INVALID_INPUT, "Resize needs scales or sizes");
    if (scales && sizes) return fail(ZANT_E_INVALID_INPUT, "Resize takes scales or sizes, not both");
    if ((scales ? nsc : nsz) != r) return fail(ZANT_E_INVALID_INPUT, "scales/sizes length != rank");
    for (size_t i = 0; i < r; ++i)
        out[i] = scales ? (size_t)std::floor((float)xs[i] * scales[i]) : sizes[i];
    return ZANT_OK;
}

// Source index of every output coordinate along every axis, computed exactly as
// nearest_interpolation does (lib_shape_math.zig:130-143): fp32 coordinate transform,
// round half away from zero, clamp.  The table is laid out axis after axis.
inline void resize_index_table(const size_t* xs, const size_t* os, size_t r, int coord_mode,
                               std::vector<int32_t>& table, std::vector<int32_t>& axis_offset) {
    table.clear(); axis_offset.assign(r, 0);
    for (size_t i = 0; i < r; ++i) {
        axis_offset[i] = (int32_t)table.size();
        const float scale = (float)os[i] / (float)xs[i];
        for (size_t o = 0; o < os[i]; ++o) {
            float pos;
            if (coord_mode == 0) pos = ((float)o + 0.5f) / scale - 0.5f;
            else if (coord_mode == 1) pos = (float)o * (float)(xs[i] - 1) / (float)(os[i] - 1);
            else pos = (float)o / scale;
            const int32_t idx = (int32_t)std::roundf(pos);
            table.push_back(std::min(std::max(idx, 0), (int32_t)(xs[i] - 1)));
        }
    }
}

inline int coord_mode_code(const char* s, size_t len) {
    if (bytes_eq(s, len, "half_pixel")) return 0;
    if (bytes_eq(s, len, "align_corners")) return 1;
    return 2;  // asymmetric
}

// ------------------------------------------------------------------------------------ reshape
// reshape_lean + reshape_lean_common, lib_shape_math.zig:1139-1209.
inline int32_t reshape_resolve(const size_t* xs, size_t xr, const size_t* ns, size_t nr, size_t* out) {
    const size_t total = numel(xs, xr);
    long long wildcard = -1;
    size_t known = 1;
    for (size_t i = 0; i < nr; ++i) {
        if (ns[i] == 0) {
            if (i >= xr) return fail(ZANT_E_INVALID_INPUT, "0 at position %zu beyond input rank", i);
            out[i] = xs[i]; known *= xs[i];
        } else if (ns[i] == std::numeric_limits<size_t>::max()) {
            if (wildcard >= 0) return fail(ZANT_E_INVALID_INPUT, "more than one -1");
            wildcard = (long long)i; out[i] = 1;
        } else {
            out[i] = ns[i]; known *= ns[i];
        }
    }
    if (wildcard >= 0) {
        if (known == 0) return fail(ZANT_E_INVALID_INPUT, "-1 with a zero-sized known product");
        if (total % known != 0) return fail(ZANT_E_INPUT_ARRAY_WRONG_SIZE, "%zu elements not divisible by %zu", total, known);
        out[wildcard] = total / known;
    }
    if (numel(out, nr) != total) return fail(ZANT_E_INPUT_ARRAY_WRONG_SIZE, "new shape holds %zu elements, input %zu", numel(out, nr), total);
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ reduce_mean
struct ReduceGeom {
    int mode;               // 0 = identity copy, 1 = all elements into one, 2 = axes
    size_t total, out_total, count;
    int n_keep, n_red;
    size_t keep_ostride[8], keep_istride[8];   // decode an output index into an input base offset
    size_t red_size[8], red_istride[8];        // reduced dims, fastest-varying first
};

// lean_reduce_mean, lib_reduction_math.zig:87-268.
inline int32_t reduce_resolve(const size_t* xs, size_t xr, const size_t* ys, size_t yr,
                              const int64_t* axes, size_t na, bool noop, ReduceGeom& g) {
    g.total = numel(xs, xr);
    g.out_total = numel(ys, yr);
    if (xr > 8) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "rank %zu", xr);
    if (!axes || na == 0) {
        g.mode = noop ? 0 : 1;
        g.count = g.total;
        if (noop && g.out_total != g.total) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "identity ReduceMean needs equal sizes");
        if (!noop && g.out_total < 1) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "empty output");
        return ZANT_OK;
    }
    if (na > 8) return fail(ZANT_E_INVALID_AXES, "too many axes");
    size_t ax[8];
    for (size_t i = 0; i < na; ++i) {
        const int64_t a = axes[i] < 0 ? axes[i] + (int64_t)xr : axes[i];
        if (a < 0 || a >= (int64_t)xr) return fail(ZANT_E_INVALID_AXES, "axis %lld for rank %zu", (long long)axes[i], xr);
        ax[i] = (size_t)a;
    }
    size_t istr[8], s = 1;
    for (size_t d = xr; d-- > 0;) { istr[d] = s; s *= xs[d]; }
    g.mode = 2; g.count = 1; g.n_red = (int)na; g.n_keep = 0;
    for (size_t i = 0; i < na; ++i) {
        g.count *= xs[ax[i]];
        g.red_size[na - 1 - i] = xs[ax[i]];      // last listed axis varies fastest (:239-257)
        g.red_istride[na - 1 - i] = istr[ax[i]];
    }
    size_t keep[8];
    for (size_t d = 0; d < xr; ++d)
        if (std::find(ax, ax + na, d) == ax + na) keep[g.n_keep++] = d;
    s = 1;
    for (int i = g.n_keep; i-- > 0;) { g.keep_ostride[i] = s; g.keep_istride[i] = istr[keep[i]]; s *= xs[keep[i]]; }
    if (g.out_total != s) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output holds %zu elements, expected %zu", g.out_total, s);
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ sharding
inline int32_t shard_range(size_t total, size_t world, size_t rank, size_t* begin, size_t* count) {
    if (world == 0 || rank >= world) return fail(ZANT_E_INVALID_INPUT, "rank %zu of %zu", rank, world);
    const size_t base = total / world, extra = total % world;
    *count = base + (rank < extra ? 1 : 0);
    *begin = rank * base + std::min(rank, extra);
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------------
// Transpose / Slice / Gather: all three are "output element i comes from input element f(i)" with f
// affine in the output coordinates (plus one table look-up for Gather).
// ------------------------------------------------------------------------------------------
struct StridedMap {
    int rank = 0;
    long long out_dims[8] = {0};
    long long in_stride[8] = {0};   // elements; may be negative (Slice with a negative step)
    long long base = 0;
    size_t total = 0;
};

// transpose_onnx_lean, lib_shape_math.zig:1628-1700.
inline int32_t transpose_resolve(const size_t* xs, size_t xr, const size_t* perm, size_t np, const size_t* ys, size_t yr, StridedMap& m) {
    if (xr > 8) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "rank %zu", xr);
    if (yr != xr) return fail(ZANT_E_INVALID_RANK, "output rank %zu, input rank %zu", yr, xr);
    size_t rp[8];
    if (perm) {
        if (np != xr) return fail(ZANT_E_INVALID_PERMUTATION, "perm holds %zu entries for rank %zu", np, xr);
        bool used[8] = {false};
        for (size_t i = 0; i < xr; ++i) {
            if (perm[i] >= xr || used[perm[i]]) return fail(ZANT_E_INVALID_PERMUTATION, "perm[%zu] = %zu", i, perm[i]);
            used[perm[i]] = true;
            rp[i] = perm[i];
        }
    } else {
        for (size_t i = 0; i < xr; ++i) rp[i] = xr - 1 - i;
    }
    long long istr[8], st = 1;
    for (size_t i = xr; i-- > 0;) { istr[i] = st; st *= (long long)xs[i]; }
    m.rank = (int)xr; m.base = 0; m.total = 1;
    for (size_t d = 0; d < xr; ++d) {
        m.out_dims[d] = (long long)xs[rp[d]];
        m.in_stride[d] = istr[rp[d]];
        if (ys[d] != xs[rp[d]]) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output dim %zu is %zu, expected %zu", d, ys[d], xs[rp[d]]);
        m.total *= xs[rp[d]];
    }
    return ZANT_OK;
}

// get_slice_output_shape (lib_shape_math.zig:1497-1560) and lean_slice_onnx (:1378-1443) normalise
// starts / ends / steps identically but count the elements of a NEGATIVE step differently: the shape
// function takes (start - end) / |step| + 1, the operator ceil((start - end - 1) / |step|) and then writes
// its own count into the output's shape.  `shape_rule` selects the former.  `out_dims` gets xr entries.
inline int32_t slice_resolve(const size_t* xs, size_t xr, const int64_t* starts, const int64_t* ends, size_t n, const int64_t* axes,
                             const int64_t* steps, size_t* out_dims, StridedMap* m, bool shape_rule = false) {
    if (xr > 8) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "rank %zu", xr);
    long long a_start[8], a_end[8], a_step[8];
    for (size_t i = 0; i < xr; ++i) { a_start[i] = 0; a_end[i] = (long long)xs[i]; a_step[i] = 1; }
    for (size_t i = 0; i < n; ++i) {
        const long long axis = axes ? axes[i] : (long long)i;
        const long long ax = axis < 0 ? axis + (long long)xr : axis;
        if (ax < 0 || (size_t)ax >= xr) return fail(ZANT_E_INVALID_SLICE_INDICES, "axis %lld for rank %zu", axis, xr);
        const long long dim = (long long)xs[ax];
        long long s0 = starts[i] < 0 ? starts[i] + dim : starts[i];
        s0 = std::max(0LL, std::min(s0, dim));
        long long e0 = ends[i] < 0 ? ends[i] + dim : ends[i];
        if (steps && steps[i] < 0) e0 = ends[i] < 0 ? -1 : e0;
        else e0 = std::max(0LL, std::min(e0, dim));
        a_start[ax] = s0; a_end[ax] = e0;
        if (steps) {
            if (steps[i] == 0) return fail(ZANT_E_INVALID_SLICE_STEP, "step 0 on axis %lld", axis);
            a_step[ax] = steps[i];
        }
    }
    long long istr[8], st = 1;
    for (size_t i = xr; i-- > 0;) { istr[i] = st; st *= (long long)xs[i]; }
    if (m) { m->rank = (int)xr; m->base = 0; m->total = 1; }
    for (size_t i = 0; i < xr; ++i) {
        long long d = 0;
        if (a_step[i] > 0) { if (a_end[i] > a_start[i]) d = ((a_end[i] - a_start[i]) + a_step[i] - 1) / a_step[i]; }
        else if (a_start[i] > a_end[i]) {
            const long long as = -a_step[i];
            if (shape_rule) d = (a_start[i] - a_end[i]) / as + 1;
            else { const long long range = a_start[i] - (a_end[i] + 1); d = (range + as - 1) / as; }
        }
        out_dims[i] = (size_t)d;
        if (m) { m->out_dims[i] = d; m->in_stride[i] = a_step[i] * istr[i]; m->base += a_start[i] * istr[i]; m->total *= (size_t)d; }
    }
    return ZANT_OK;
}

struct GatherGeom { size_t outer = 0, n_idx = 0, inner = 0, axis_dim = 0; };

// gather, lib_shape_math.zig:1217-1277 (validation and output shape) over host indices.
inline int32_t gather_resolve(const size_t* xs, size_t xr, const size_t* indices, const size_t* is, size_t ir, int64_t axis_in,
                              const size_t* ys, size_t yr, GatherGeom& g) {
    if (xr == 0) return fail(ZANT_E_INVALID_RANK, "gather on a rank-0 tensor");
    const long long nd = (long long)xr;
    if (axis_in >= nd || axis_in < -nd) return fail(ZANT_E_INVALID_AXIS, "axis %lld for rank %zu", (long long)axis_in, xr);
    const size_t axis = (size_t)(axis_in < 0 ? nd + axis_in : axis_in);
    g.n_idx = 1;
    for (size_t i = 0; i < ir; ++i) g.n_idx *= is[i];
    for (size_t i = 0; i < g.n_idx; ++i)
        if (indices[i] >= xs[axis]) return fail(ZANT_E_INDEX_OUT_OF_BOUNDS, "index %zu on an axis of %zu", indices[i], xs[axis]);
    if (yr != xr + ir - 1) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output rank %zu, expected %zu", yr, xr + ir - 1);
    bool ok = true;
    for (size_t i = 0; i < axis; ++i) ok = ok && ys[i] == xs[i];
    for (size_t i = 0; i < ir; ++i) ok = ok && ys[axis + i] == is[i];
    for (size_t i = axis + 1; i < xr; ++i) ok = ok && ys[axis + ir + (i - axis - 1)] == xs[i];
    if (!ok) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "gather output shape");
    g.outer = 1; g.inner = 1; g.axis_dim = xs[axis];
    for (size_t i = 0; i < axis; ++i) g.outer *= xs[i];
    for (size_t i = axis + 1; i < xr; ++i) g.inner *= xs[i];
    return ZANT_OK;
}

}  // namespace zb
