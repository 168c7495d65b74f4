// Device-level operator launchers: resolved geometry + device pointers -> kernel launches on
// the context's stream.  Shared by the single-operator C entry points and by the plan.
#pragma once
#include <type_traits>
#include "context.cuh"
#include "geometry.hpp"
#include "kernels_f32.cuh"
#include "kernels_q8.cuh"

namespace zb {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------------------- fp32
inline int32_t run_conv_f32(zant_ctx* ctx, const ConvGeom& g, const float* x, const float* w, const float* bias, float* y) {
    ContractArgs p{};
    p.a = x; p.b = w; p.d = y; p.bias = bias; p.g = g;
    const long long M = (long long)g.N * g.OH * g.OW;
    if (M > 0x7fffffffLL) return fail(ZANT_E_TOO_LARGE, "Conv output pixels exceed int range");
    p.M = (int)M; p.N = g.M; p.K = g.C * g.KH * g.KW;
    dim3 grid((p.M + CT_BM - 1) / CT_BM, (p.N + CT_BN - 1) / CT_BN);
    if (grid.y > 65535) return fail(ZANT_E_TOO_LARGE, "too many output channels");
    contract_f32_exact<true><<<grid, 256, 0, ctx->stream>>>(p);
    return check_launch(ctx, "contract_f32_exact<conv>");
}

inline int32_t run_contract_f32(zant_ctx* ctx, ContractArgs& p) {
    dim3 grid((p.M + CT_BM - 1) / CT_BM, (p.N + CT_BN - 1) / CT_BN);
    if (grid.y > 65535) return fail(ZANT_E_TOO_LARGE, "too many output columns");
    contract_f32_exact<false><<<grid, 256, 0, ctx->stream>>>(p);
    return check_launch(ctx, "contract_f32_exact<matrix>");
}

inline int32_t run_matmul_f32(zant_ctx* ctx, const MatGeom& g, const float* a, const float* b, float* y) {
    if (g.M > 0x7fffffffULL || g.N > 0x7fffffffULL || g.K > 0x7fffffffULL) return fail(ZANT_E_TOO_LARGE, "MatMul dims exceed int range");
    ContractArgs p{};
    p.a = a; p.b = b; p.d = y; p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
    p.sam = (long long)g.K; p.sak = 1; p.sbk = (long long)g.N; p.sbj = 1;
    return run_contract_f32(ctx, p);
}

inline int32_t run_gemm_f32(zant_ctx* ctx, const GemmGeom& g, const float* a, const float* b, const float* c,
                            float alpha, float beta, bool ta, bool tb, float* y) {
    if (g.rows > 0x7fffffffULL || g.cols > 0x7fffffffULL || g.K > 0x7fffffffULL) return fail(ZANT_E_TOO_LARGE, "Gemm dims exceed int range");
    ContractArgs p{};
    p.a = a; p.b = b; p.d = y; p.M = (int)g.rows; p.N = (int)g.cols; p.K = (int)g.K;
    // A' = A^T when transA: A is [K, rows] row-major; B' = B^T when transB: B is [cols, K].
    p.sam = ta ? 1 : (long long)g.K; p.sak = ta ? (long long)g.rows : 1;
    p.sbk = tb ? 1 : (long long)g.cols; p.sbj = tb ? (long long)g.K : 1;
    p.epilogue = 1; p.alpha = alpha; p.beta = beta; p.c = c; p.c_mode = g.c_mode;
    if (g.c_mode == 1) { p.c_rs = (long long)g.cols; p.c_cs = 1; }
    else if (g.c_mode == 2) { p.c_rs = g.c_rows == 1 ? 0 : (long long)g.c_cols; p.c_cs = g.c_cols == 1 ? 0 : 1; }
    int32_t st = run_contract_f32(ctx, p);
    if (st != ZANT_OK) return st;
    const size_t first = g.rows * g.cols, total = g.batch * first;
    if (total > first) {
        gemm_tail_f32<<<grid_for(total - first, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
            y, first, total, alpha, c, g.c_mode, beta, g.rows, g.cols, g.c_rows, g.c_cols, 0, g.c_ch);
        st = check_launch(ctx, "gemm_tail_f32");
    }
    return st;
}

template <typename T>
inline int32_t run_maxpool(zant_ctx* ctx, const PoolGeom& g, const T* x, T* y) {
    const size_t total = (size_t)g.NC * g.OH * g.OW;
    if (total == 0) return ZANT_OK;
    if constexpr (sizeof(T) == 1) {
        const bool fast = g.KH == 2 && g.KW == 2 && g.sh == 2 && g.sw == 2 && g.dh == 1 && g.dw == 1 && g.pt == 0 && g.pl == 0 &&
                          g.W % 8 == 0 && g.H == 2 * g.OH && g.W == 2 * g.OW &&
                          (reinterpret_cast<uintptr_t>(x) & 7u) == 0 && (reinterpret_cast<uintptr_t>(y) & 3u) == 0;
        if (fast) {
            const size_t words = total / 4;
            const int grid = grid_for(words, 256, ctx->sm_count, 16);
            if (std::is_signed<T>::value)
                maxpool2x2s2_q8<true><<<grid, 256, 0, ctx->stream>>>((const uint2*)x, (uint32_t*)y, (size_t)g.NC * g.OH, g.OW / 4, g.W / 8);
            else
                maxpool2x2s2_q8<false><<<grid, 256, 0, ctx->stream>>>((const uint2*)x, (uint32_t*)y, (size_t)g.NC * g.OH, g.OW / 4, g.W / 8);
            return check_launch(ctx, "maxpool2x2s2_q8");
        }
    }
    if constexpr (std::is_same<T, float>::value) {
        const bool fast = g.KH == 2 && g.KW == 2 && g.sh == 2 && g.sw == 2 && g.dh == 1 && g.dw == 1 && g.pt == 0 && g.pl == 0 &&
                          g.W % 4 == 0 && g.H == 2 * g.OH && g.W == 2 * g.OW &&
                          (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(y) & 7u) == 0;
        if (fast) {
            const size_t pairs = total / 2;
            maxpool2x2s2_f32<<<grid_for(pairs, 256, ctx->sm_count, 16), 256, 0, ctx->stream>>>((const float4*)x, (float2*)y, (size_t)g.NC * g.OH, g.OW / 2, g.W / 4);
            return check_launch(ctx, "maxpool2x2s2_f32");
        }
    }
    maxpool_nchw<T><<<grid_for(total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(x, y, g);
    return check_launch(ctx, "maxpool_nchw");
}

template <typename F>
inline int32_t run_unary_f32(zant_ctx* ctx, const float* x, float* y, size_t n, F f, const char* name) {
    if (n == 0) return ZANT_OK;
    const bool vec = aligned16(x) && aligned16(y);
    unary_f32<F><<<grid_for(vec ? (n + 3) / 4 : n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(x, y, n, vec, f);
    return check_launch(ctx, name);
}

inline int32_t run_binary_same_f32(zant_ctx* ctx, const float* a, const float* b, float* y, size_t n, bool divide) {
    if (n == 0) return ZANT_OK;
    const int grid = grid_for(n, 256, ctx->sm_count);
    if (divide) binary_same_f32<true><<<grid, 256, 0, ctx->stream>>>(a, b, y, n);
    else binary_same_f32<false><<<grid, 256, 0, ctx->stream>>>(a, b, y, n);
    return check_launch(ctx, divide ? "div_f32" : "mul_f32");
}

inline int32_t run_softmax_f32(zant_ctx* ctx, const float* x, float* y, size_t rows, size_t cols) {
    if (rows == 0 || cols == 0) return ZANT_OK;
    softmax_rows_f32<<<grid_for(rows, 128, ctx->sm_count), 128, 0, ctx->stream>>>(x, y, rows, cols);
    return check_launch(ctx, "softmax_rows_f32");
}

inline int32_t run_add_f32(zant_ctx* ctx, const BcastGeom& g, const float* a, const float* b, float* y) {
    if (g.total == 0) return ZANT_OK;
    if (g.same_size) {
        const bool vec = aligned16(a) && aligned16(b) && aligned16(y);
        add_same_f32<<<grid_for(vec ? (g.total + 3) / 4 : g.total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(a, b, y, g.total, vec);
        return check_launch(ctx, "add_same_f32");
    }
    BcastArgs k{};
    k.rank = g.rank; k.total = g.total;
    for (int d = 0; d < g.rank; ++d) { k.out_shape[d] = g.out_shape[d]; k.a_stride[d] = g.a_stride[d]; k.b_stride[d] = g.b_stride[d]; }
    add_bcast_f32<<<grid_for(g.total, 256, ctx->sm_count), 256, 0, ctx->stream>>>(a, b, y, k);
    return check_launch(ctx, "add_bcast_f32");
}

inline int32_t run_sum_list_f32(zant_ctx* ctx, const float* const* ts, size_t nt, float* y, size_t n) {
    if (n == 0) return ZANT_OK;
    size_t done = 0;
    while (done < nt) {
        SumListArgs l{};
        l.n = (int)std::min<size_t>(8, nt - done);
        for (int i = 0; i < l.n; ++i) l.t[i] = ts[done + i];
        sum_list_f32<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(l, y, n, done != 0);
        int32_t st = check_launch(ctx, "sum_list_f32");
        if (st != ZANT_OK) return st;
        done += l.n;
    }
    return ZANT_OK;
}

inline int32_t run_copy2d(zant_ctx* ctx, const void* src, size_t sp, void* dst, size_t dp, size_t row_bytes, size_t rows) {
    if (row_bytes == 0 || rows == 0) return ZANT_OK;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | sp | dp | row_bytes;
    const char* s = static_cast<const char*>(src);
    char* d = static_cast<char*>(dst);
    if ((bits & 15) == 0) {
        copy2d<uint4><<<grid_for(row_bytes / 16 * rows, 256, ctx->sm_count), 256, 0, ctx->stream>>>(s, sp, d, dp, row_bytes / 16, rows);
    } else if ((bits & 3) == 0) {
        copy2d<uint32_t><<<grid_for(row_bytes / 4 * rows, 256, ctx->sm_count), 256, 0, ctx->stream>>>(s, sp, d, dp, row_bytes / 4, rows);
    } else {
        copy2d<uint8_t><<<grid_for(row_bytes * rows, 256, ctx->sm_count), 256, 0, ctx->stream>>>(s, sp, d, dp, row_bytes, rows);
    }
    return check_launch(ctx, "copy2d");
}

// One strided copy per input tensor: slice s of tensor t lands at out[s*out_row + off_t].
inline int32_t run_concat(zant_ctx* ctx, const ConcatGeom& g, size_t esz, const void* const* ts, void* y) {
    const size_t out_row = g.out_axis_dim * g.slice * esz;
    size_t off = 0;
    for (size_t t = 0; t < g.axis_dim.size(); ++t) {
        const size_t row = g.axis_dim[t] * g.slice * esz;
        int32_t st = run_copy2d(ctx, ts[t], row, static_cast<char*>(y) + off, out_row, row, g.num_slices);
        if (st != ZANT_OK) return st;
        off += row;
    }
    return ZANT_OK;
}

inline int32_t run_resize(zant_ctx* ctx, size_t esz, const void* x, void* y, const int32_t* table_dev,
                          const size_t* xs, const size_t* os, size_t r, const std::vector<int32_t>& axis_offset) {
    ResizeArgs k{};
    k.rank = (int)r; k.total = 1;
    size_t s = 1;
    for (size_t d = r; d-- > 0;) { k.in_stride[d] = s; s *= xs[d]; k.out_shape[d] = os[d]; k.total *= os[d]; k.axis_offset[d] = axis_offset[d]; }
    if (k.total == 0) return ZANT_OK;
    const int grid = grid_for(k.total, 256, ctx->sm_count);
    const bool small = k.total < 0x7fffffffull && s < 0x7fffffffull;      // s: elements of the input
    if (esz == 4) {
        if (small) resize_gather<uint32_t, uint32_t><<<grid, 256, 0, ctx->stream>>>((const uint32_t*)x, (uint32_t*)y, table_dev, k);
        else resize_gather<uint32_t, size_t><<<grid, 256, 0, ctx->stream>>>((const uint32_t*)x, (uint32_t*)y, table_dev, k);
    } else {
        if (small) resize_gather<uint8_t, uint32_t><<<grid, 256, 0, ctx->stream>>>((const uint8_t*)x, (uint8_t*)y, table_dev, k);
        else resize_gather<uint8_t, size_t><<<grid, 256, 0, ctx->stream>>>((const uint8_t*)x, (uint8_t*)y, table_dev, k);
    }
    return check_launch(ctx, "resize_gather");
}

inline int32_t run_reduce_mean_f32(zant_ctx* ctx, const ReduceGeom& g, const float* x, float* y) {
    if (g.mode == 0) {
        ZB_CUDA(cudaMemcpyAsync(y, x, g.total * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        return ZANT_OK;
    }
    if (g.mode == 1) {
        reduce_all_mean_f32<<<1, 32, 0, ctx->stream>>>(x, y, g.total);
        return check_launch(ctx, "reduce_all_mean_f32");
    }
    ReduceArgs k{};
    k.out_total = g.out_total; k.count = g.count; k.n_keep = g.n_keep; k.n_red = g.n_red;
    for (int i = 0; i < 8; ++i) { k.keep_ostride[i] = g.keep_ostride[i]; k.keep_istride[i] = g.keep_istride[i]; k.red_size[i] = g.red_size[i]; k.red_istride[i] = g.red_istride[i]; }
    if (g.out_total == 0) return ZANT_OK;
    reduce_mean_f32<<<grid_for(g.out_total, 128, ctx->sm_count), 128, 0, ctx->stream>>>(x, y, k);
    return check_launch(ctx, "reduce_mean_f32");
}

// ---------------------------------------------------------------------------- quantized
inline int32_t run_quantize(zant_ctx* ctx, const float* x, void* y, size_t n, float scale, int zp, int32_t out_dtype) {
    if (n == 0) return ZANT_OK;
    const bool vec = aligned16(x) && ((reinterpret_cast<uintptr_t>(y) & 3) == 0);
    const int grid = grid_for(vec ? (n + 3) / 4 : n, 256, ctx->sm_count);
    if (out_dtype == ZANT_U8) quantize_linear_k<true><<<grid, 256, 0, ctx->stream>>>(x, y, n, scale, zp, vec);
    else quantize_linear_k<false><<<grid, 256, 0, ctx->stream>>>(x, y, n, scale, zp, vec);
    return check_launch(ctx, "quantize_linear_k");
}

inline int32_t run_dequantize(zant_ctx* ctx, int32_t in_dtype, const void* q, float* y, size_t n, float scale, int zp) {
    if (n == 0) return ZANT_OK;
    const int grid = grid_for(n, 256, ctx->sm_count);
    if (in_dtype == ZANT_U8) dequantize_linear_k<uint8_t><<<grid, 256, 0, ctx->stream>>>((const uint8_t*)q, y, n, scale, zp);
    else if (in_dtype == ZANT_I8) dequantize_linear_k<int8_t><<<grid, 256, 0, ctx->stream>>>((const int8_t*)q, y, n, scale, zp);
    else dequantize_linear_k<int32_t><<<grid, 256, 0, ctx->stream>>>((const int32_t*)q, y, n, scale, zp);
    return check_launch(ctx, "dequantize_linear_k");
}

inline int32_t run_qconv_generic(zant_ctx* ctx, const QConvArgs& p, int32_t x_dtype, int32_t y_dtype) {
    const size_t total = (size_t)p.g.N * p.g.M * p.g.OH * p.g.OW;
    if (total == 0) return ZANT_OK;
    const int grid = grid_for(total, 128, ctx->sm_count, 32);
    const bool xu = x_dtype == ZANT_U8, yu = y_dtype == ZANT_U8;
    if (xu && yu) qconv_nchw_generic<true, true><<<grid, 128, 0, ctx->stream>>>(p);
    else if (xu) qconv_nchw_generic<true, false><<<grid, 128, 0, ctx->stream>>>(p);
    else if (yu) qconv_nchw_generic<false, true><<<grid, 128, 0, ctx->stream>>>(p);
    else qconv_nchw_generic<false, false><<<grid, 128, 0, ctx->stream>>>(p);
    return check_launch(ctx, "qconv_nchw_generic");
}

inline int32_t run_qmatmul_generic(zant_ctx* ctx, const QMatArgs& p, int32_t a_dtype, int32_t y_dtype) {
    const size_t total = (size_t)p.M * p.N;
    if (total == 0) return ZANT_OK;
    const int grid = grid_for(total, 128, ctx->sm_count, 32);
    const bool au = a_dtype == ZANT_U8, yu = y_dtype == ZANT_U8;
    if (au && yu) qmatmul_generic<true, true><<<grid, 128, 0, ctx->stream>>>(p);
    else if (au) qmatmul_generic<true, false><<<grid, 128, 0, ctx->stream>>>(p);
    else if (yu) qmatmul_generic<false, true><<<grid, 128, 0, ctx->stream>>>(p);
    else qmatmul_generic<false, false><<<grid, 128, 0, ctx->stream>>>(p);
    return check_launch(ctx, "qmatmul_generic");
}

inline int32_t run_qadd(zant_ctx* ctx, int32_t dtype, const void* a, float a_s, int a_zp, const void* b, float b_s, int b_zp,
                        float y_s, int y_zp, int act, void* y, size_t n) {
    if (n == 0) return ZANT_OK;
    const bool u8 = dtype == ZANT_U8;
    const bool zp_ok = u8 ? (y_zp >= 0 && y_zp <= 255) : (y_zp >= -128 && y_zp <= 127);
    size_t done = 0;
    if (zp_ok && n >= 16 && aligned16(a) && aligned16(b) && aligned16(y)) {
        const size_t n16 = n / 16;
        const int grid = grid_for(n16, 256, ctx->sm_count);
        if (u8) qadd_vec_k<true><<<grid, 256, 0, ctx->stream>>>((const uint4*)a, a_s, a_zp, (const uint4*)b, b_s, b_zp, y_s, y_zp, act, (uint4*)y, n16);
        else qadd_vec_k<false><<<grid, 256, 0, ctx->stream>>>((const uint4*)a, a_s, a_zp, (const uint4*)b, b_s, b_zp, y_s, y_zp, act, (uint4*)y, n16);
        ZB_TRY(check_launch(ctx, "qadd_vec_k"));
        done = n16 * 16;
        if (done == n) return ZANT_OK;
    }
    const char* pa = (const char*)a + done; const char* pb = (const char*)b + done; char* py = (char*)y + done;
    const size_t rest = n - done;
    const int grid = grid_for(rest, 256, ctx->sm_count);
    if (u8) qadd_k<true><<<grid, 256, 0, ctx->stream>>>(pa, a_s, a_zp, pb, b_s, b_zp, y_s, y_zp, act, py, rest);
    else qadd_k<false><<<grid, 256, 0, ctx->stream>>>(pa, a_s, a_zp, pb, b_s, b_zp, y_s, y_zp, act, py, rest);
    return check_launch(ctx, "qadd_k");
}

inline int32_t run_qgap(zant_ctx* ctx, int32_t dtype, const void* x, void* y, size_t planes, int hw,
                        float x_s, int x_zp, float y_s, int y_zp) {
    if (planes == 0) return ZANT_OK;
    if (hw <= 256 && planes >= 4096 && (reinterpret_cast<uintptr_t>(x) & 3u) == 0) {
        // many small planes: a thread per plane
        const int grid = grid_for(planes, 128, ctx->sm_count);
        if (dtype == ZANT_U8) qgap_small_k<true><<<grid, 128, 0, ctx->stream>>>((const uint8_t*)x, y, planes, hw, x_s, x_zp, y_s, y_zp);
        else qgap_small_k<false><<<grid, 128, 0, ctx->stream>>>((const uint8_t*)x, y, planes, hw, x_s, x_zp, y_s, y_zp);
        return check_launch(ctx, "qgap_small_k");
    }
    const int grid = grid_for(planes * 32, 256, ctx->sm_count);
    if (dtype == ZANT_U8) qgap_k<true><<<grid, 256, 0, ctx->stream>>>(x, y, planes, hw, x_s, x_zp, y_s, y_zp);
    else qgap_k<false><<<grid, 256, 0, ctx->stream>>>(x, y, planes, hw, x_s, x_zp, y_s, y_zp);
    return check_launch(ctx, "qgap_k");
}

inline int32_t run_lut(zant_ctx* ctx, const void* x, void* y, size_t n, const uint8_t* lut_dev) {
    if (n == 0) return ZANT_OK;
    const bool vec = aligned16(x) && aligned16(y);
    lut_q8_k<<<grid_for(vec ? (n + 15) / 16 : n, 256, ctx->sm_count), 256, 0, ctx->stream>>>((const uint8_t*)x, (uint8_t*)y, n, lut_dev, vec);
    return check_launch(ctx, "lut_q8_k");
}

// Per-output-channel requantisation multipliers M[m] = (x_scale * w_scale[m]) / y_scale:
// one fp32 multiply then one fp32 divide, computed on the host once.
inline void requant_multipliers(float x_scale, const float* w_scale, size_t nws, float y_scale, size_t M, std::vector<float>& out) {
    out.resize(M);
    for (size_t m = 0; m < M; ++m) {
        volatile float xw = x_scale * w_scale[nws == 1 ? 0 : m];
        out[m] = xw / y_scale;
    }
}

inline int32_t run_strided_copy(zant_ctx* ctx, size_t esz, const void* x, void* y, const StridedMap& m) {
    if (m.total == 0) return ZANT_OK;
    StridedMapDev d{};
    d.rank = m.rank; d.base = m.base; d.total = m.total;
    for (int i = 0; i < 8; ++i) { d.out_dims[i] = m.out_dims[i]; d.in_stride[i] = m.in_stride[i]; }
    const int grid = grid_for(m.total, 256, ctx->sm_count);
    if (esz == 4) strided_copy_k<uint32_t><<<grid, 256, 0, ctx->stream>>>((const uint32_t*)x, (uint32_t*)y, d);
    else strided_copy_k<uint8_t><<<grid, 256, 0, ctx->stream>>>((const uint8_t*)x, (uint8_t*)y, d);
    return check_launch(ctx, "strided_copy_k");
}

inline int32_t run_gather(zant_ctx* ctx, size_t esz, const void* x, const int32_t* idx_dev, void* y, const GatherGeom& g) {
    const size_t total = g.outer * g.n_idx * g.inner;
    if (total == 0) return ZANT_OK;
    const int grid = grid_for(total, 256, ctx->sm_count);
    if (esz == 4) gather_axis_k<uint32_t><<<grid, 256, 0, ctx->stream>>>((const uint32_t*)x, idx_dev, (uint32_t*)y, g.outer, g.n_idx, g.inner, g.axis_dim);
    else gather_axis_k<uint8_t><<<grid, 256, 0, ctx->stream>>>((const uint8_t*)x, idx_dev, (uint8_t*)y, g.outer, g.n_idx, g.inner, g.axis_dim);
    return check_launch(ctx, "gather_axis_k");
}

}  // namespace zb
