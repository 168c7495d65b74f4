// extern "C" entry points declared in include/zant_b200.h: argument checks (host), staging of
// host buffers, kernel launches.  No entry point has a CPU implementation: without a context
// (i.e. without a usable GPU) every compute call returns ZANT_E_CUDA_UNAVAILABLE after its
// arguments have been validated.
#include <cuda_runtime.h>

#include <cstdint>
#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/zant_b200.h"
#include "context.cuh"
#include "geometry.hpp"
#include "ops.cuh"
#include "tc_peak.cuh"
#include "selftest.cuh"
#include "tc_gemm_tf32.cuh"
#include "tc_conv_generic.cuh"
#include "tc_conv_nchw.cuh"
#include "tc_pw_nchw.cuh"
#include "dwconv_q8.cuh"
#include "smallc_conv_q8.cuh"
#include "tc_conv_nhwc.cuh"
#include "status.hpp"

using namespace zb;

#define ZB_NEED(ptr, what) \
    do { if ((ptr) == nullptr) return fail(ZANT_E_NULL_POINTER, "%s is NULL", what); } while (0)

#define ZB_NEED_CTX(ctx)                                                                                     \
    do {                                                                                                     \
        if ((ctx) == nullptr) return fail(ZANT_E_CUDA_UNAVAILABLE, "no context (zant_b200_ctx_create failed or was not called); there is no CPU fallback"); \
        ZB_CUDA(cudaSetDevice((ctx)->device));                                                               \
    } while (0)


extern "C" {

// ------------------------------------------------------------------------------------ library / context
const char* zant_b200_version(void) { return "zant-b200 0.1 (sm_100a)"; }
const char* zant_b200_status_name(int32_t status) { return status_name(status); }
const char* zant_b200_last_error(void) { return last_error_ref().c_str(); }
void zant_b200_set_log(void (*fn)(char*)) { log_fn_ref() = fn; }

int32_t zant_b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int32_t zant_b200_ctx_create(int32_t device, size_t arena_bytes, zant_ctx** out) {
    ZB_NEED(out, "out");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(ZANT_E_CUDA_UNAVAILABLE, "no CUDA device (%s)", e != cudaSuccess ? cudaGetErrorString(e) : "count is 0");
    }
    if (device < 0 || device >= n) return fail(ZANT_E_INVALID_INPUT, "device %d of %d", device, n);
    ZB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    ZB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(ZANT_E_CUDA_UNAVAILABLE, "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
    zant_ctx* c = new zant_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete c; return fail(ZANT_E_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); }
    const size_t want = arena_bytes ? arena_bytes : (size_t)256 << 20;
    e = dev_malloc((void**)&c->arena, want);
    if (e != cudaSuccess) {
        cudaGetLastError(); cudaStreamDestroy(c->stream); delete c;
        return fail(e == cudaErrorMemoryAllocation ? ZANT_E_MEM_ERROR : ZANT_E_CUDA, "cudaMalloc(%zu): %s", want, cudaGetErrorString(e));
    }
    c->arena_bytes = want;
    e = dev_malloc((void**)&c->status_word, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->status_word, 0, sizeof(int));
    if (e != cudaSuccess) { cudaFree(c->arena); cudaStreamDestroy(c->stream); delete c; return fail(ZANT_E_CUDA, "status word: %s", cudaGetErrorString(e)); }
    if (const char* v = std::getenv("ZANT_B200_TF32")) c->tf32 = (v[0] == '2') ? 2 : (env_flag("ZANT_B200_TF32") ? 1 : 0);
    *out = c;
    log_line("zant_b200 context on device %d (%s, %d SMs)", device, prop.name, prop.multiProcessorCount);
    return ZANT_OK;
}

int32_t zant_b200_ctx_destroy(zant_ctx* ctx) {
    if (!ctx) return ZANT_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->arena) cudaFree(ctx->arena);
    if (ctx->status_word) cudaFree(ctx->status_word);
    if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return ZANT_OK;
}

int32_t zant_b200_ctx_set_stream(zant_ctx* ctx, void* cuda_stream) {
    ZB_NEED_CTX(ctx);
    ZB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->own_stream && ctx->stream) ZB_CUDA(cudaStreamDestroy(ctx->stream));
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    ctx->own_stream = false;
    return ZANT_OK;
}

int32_t zant_b200_ctx_set_tf32(zant_ctx* ctx, int32_t enable) {
    ZB_NEED_CTX(ctx);
    if (enable < 0 || enable > 2) return fail(ZANT_E_INVALID_INPUT, "TF32 mode %d (0 exact FP32, 1 TF32, 2 split TF32)", enable);
    ctx->tf32 = enable;
    return ZANT_OK;
}

int32_t zant_b200_ctx_get_tf32(zant_ctx* ctx) { return ctx ? ctx->tf32 : 0; }

int32_t zant_b200_ctx_set_arena_limit(zant_ctx* ctx, size_t max_bytes) {
    ZB_NEED_CTX(ctx);
    ctx->arena_limit = max_bytes;
    return ZANT_OK;
}

void* zant_b200_ctx_stream(zant_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int32_t zant_b200_ctx_synchronize(zant_ctx* ctx) {
    ZB_NEED_CTX(ctx);
    return drain_and_check_status(ctx);
}

uint64_t zant_b200_ctx_launch_count(zant_ctx* ctx) { return ctx ? ctx->launches : 0; }
void zant_b200_ctx_reset_launch_count(zant_ctx* ctx) { if (ctx) ctx->launches = 0; }

int32_t zant_b200_measure_int8_peak(zant_ctx* ctx, int32_t iters, double* tera_ops_per_s) {
    ZB_NEED(tera_ops_per_s, "tera_ops_per_s");
    ZB_NEED_CTX(ctx);
    if (iters < 64) iters = 64;
    if (iters > (1 << 20)) iters = 1 << 20;
    ZB_CUDA(cudaFuncSetAttribute(tc_peak_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PEAK_SMEM));
    cudaEvent_t e0, e1;
    ZB_CUDA(cudaEventCreate(&e0)); ZB_CUDA(cudaEventCreate(&e1));
    float best = 1e30f;
    for (int rep = 0; rep < 5; ++rep) {      // first repetition is the warm-up
        ZB_CUDA(cudaEventRecord(e0, ctx->stream));
        tc_peak_i8_kernel<<<ctx->sm_count, 128, PEAK_SMEM, ctx->stream>>>(iters, ctx->status_word);
        ZB_TRY(check_launch(ctx, "tc_peak_i8_kernel"));
        ZB_CUDA(cudaEventRecord(e1, ctx->stream));
        ZB_TRY(drain_and_check_status(ctx));
        float ms = 0.0f;
        ZB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    const double ops = (double)ctx->sm_count * iters * 2.0 * (2.0 * 128 * 256 * 32);
    *tera_ops_per_s = ops / (best * 1e-3) / 1e12;
    return ZANT_OK;
}

int32_t zant_b200_measure_int8_peak_sustained(zant_ctx* ctx, double seconds, double* tera_ops_per_s) {
    ZB_NEED(tera_ops_per_s, "tera_ops_per_s");
    ZB_NEED_CTX(ctx);
    if (!(seconds > 0.05)) seconds = 0.05;
    if (seconds > 10.0) seconds = 10.0;
    ZB_CUDA(cudaFuncSetAttribute(tc_peak_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PEAK_SMEM));
    const int iters = 20000;                                   // ~15 ms per launch at the burst rate
    cudaEvent_t e0, e1;
    ZB_CUDA(cudaEventCreate(&e0)); ZB_CUDA(cudaEventCreate(&e1));
    tc_peak_i8_kernel<<<ctx->sm_count, 128, PEAK_SMEM, ctx->stream>>>(iters, ctx->status_word);   // warm-up
    ZB_TRY(check_launch(ctx, "tc_peak_i8_kernel"));
    ZB_TRY(drain_and_check_status(ctx));
    // launches back to back, in batches that are timed on the device, until the requested time has passed
    double total_ms = 0.0; long long launches = 0;
    while (total_ms < seconds * 1e3) {
        ZB_CUDA(cudaEventRecord(e0, ctx->stream));
        for (int k = 0; k < 16; ++k) {
            tc_peak_i8_kernel<<<ctx->sm_count, 128, PEAK_SMEM, ctx->stream>>>(iters, ctx->status_word);
            ZB_TRY(check_launch(ctx, "tc_peak_i8_kernel"));
        }
        ZB_CUDA(cudaEventRecord(e1, ctx->stream));
        ZB_TRY(drain_and_check_status(ctx));
        float ms = 0.0f;
        ZB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        total_ms += ms; launches += 16;
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    const double ops = (double)launches * ctx->sm_count * iters * 2.0 * (2.0 * 128 * 256 * 32);
    *tera_ops_per_s = ops / (total_ms * 1e-3) / 1e12;
    return ZANT_OK;
}

int32_t zant_b200_selftest_bounded_wait(zant_ctx* ctx, uint32_t budget_us) {
    ZB_NEED_CTX(ctx);
    if (budget_us == 0) budget_us = 1;
    if (budget_us > 100000) budget_us = 100000;                 // a tenth of a second at most
    const long long cycles = (long long)budget_us * 2000;       // ~2 GHz SM clock
    bounded_wait_selftest_kernel<<<1, 64, 0, ctx->stream>>>(cycles, ctx->status_word);
    return check_launch(ctx, "bounded_wait_selftest_kernel");
}

int32_t zant_b200_debug_fail_alloc(int32_t nth) {
    alloc_failures_armed().store(nth > 0 ? nth : 0);
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ shape helpers
int32_t zant_b200_conv_output_shape(const size_t* x_shape, size_t x_rank, const size_t* w_shape, size_t w_rank,
                                    const size_t* stride, size_t n_stride, const size_t* pads, size_t n_pads,
                                    const size_t* dilations, size_t n_dil, const char* auto_pad, size_t auto_pad_len,
                                    size_t out_shape[4]) {
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(w_shape, "w_shape"); ZB_NEED(out_shape, "out_shape");
    return conv_output_shape_ref(x_shape, x_rank, w_shape, w_rank, stride, n_stride, pads, n_pads, dilations, n_dil,
                                 auto_pad, auto_pad_len, out_shape);
}

int32_t zant_b200_pooling_output_shape(const size_t* x_shape, size_t x_rank, const size_t kernel[2], const size_t stride[2],
                                       size_t out_shape[4]) {
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(kernel, "kernel"); ZB_NEED(stride, "stride"); ZB_NEED(out_shape, "out_shape");
    return pooling_output_shape(x_shape, x_rank, kernel, stride, out_shape);
}

int32_t zant_b200_maxpool_output_shape(const size_t* x_shape, size_t x_rank, const size_t* kernel_shape, const size_t* strides,
                                       const size_t* dilations, const size_t* pads, int32_t auto_pad, int32_t ceil_mode,
                                       size_t out_shape[4]) {
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(out_shape, "out_shape");
    return maxpool_output_shape(x_shape, x_rank, kernel_shape, strides, dilations, pads, auto_pad, ceil_mode, out_shape);
}

int32_t zant_b200_resize_output_shape(const size_t* x_shape, size_t rank, const float* scales, size_t n_scales,
                                      const size_t* sizes, size_t n_sizes, size_t* out_shape) {
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(out_shape, "out_shape");
    return resize_output_shape(x_shape, rank, scales, n_scales, sizes, n_sizes, out_shape);
}

int32_t zant_b200_concat_output_shape(const size_t* const* shapes, const size_t* ranks, size_t n_tensors, int64_t axis,
                                      size_t* out_shape, size_t* out_rank) {
    ZB_NEED(out_shape, "out_shape"); ZB_NEED(out_rank, "out_rank");
    if (n_tensors) { ZB_NEED(shapes, "shapes"); ZB_NEED(ranks, "ranks"); }
    ConcatGeom g;
    size_t tmp[8];
    ZB_TRY(concat_resolve(shapes, ranks, n_tensors, axis, tmp, g));
    for (size_t d = 0; d < g.rank; ++d) out_shape[d] = tmp[d];
    *out_rank = g.rank;
    return ZANT_OK;
}

int32_t zant_b200_get_concatenate_output_shape(const size_t* const* shapes, const size_t* ranks, size_t n_tensors,
                                               int64_t axis, size_t* out_shape) {
    ZB_NEED(out_shape, "out_shape");
    if (n_tensors) { ZB_NEED(shapes, "shapes"); ZB_NEED(ranks, "ranks"); }
    return concat_output_shape_strict(shapes, ranks, n_tensors, axis, out_shape);
}

int32_t zant_b200_shard_range(size_t total, size_t world, size_t rank, size_t* begin, size_t* count) {
    ZB_NEED(begin, "begin"); ZB_NEED(count, "count");
    return shard_range(total, world, rank, begin, count);
}

// ------------------------------------------------------------------------------------ fp32 operators
int32_t zant_b200_conv_f32(zant_ctx* ctx, const float* x, const size_t* x_shape, size_t x_rank,
                           const float* w, const size_t* w_shape, size_t w_rank, const float* bias, size_t bias_len,
                           float* y, const size_t* y_shape, size_t y_rank,
                           const size_t* stride, size_t n_stride, const size_t* pads, size_t n_pads,
                           const size_t* dilations, size_t n_dil, size_t group, const char* auto_pad, size_t auto_pad_len) {
    ZB_NEED(x, "x"); ZB_NEED(w, "w"); ZB_NEED(y, "y"); ZB_NEED(x_shape, "x_shape"); ZB_NEED(w_shape, "w_shape"); ZB_NEED(y_shape, "y_shape");
    ConvGeom g;
    ZB_TRY(conv_resolve_ref(x_shape, x_rank, w_shape, w_rank, y_shape, y_rank, stride, n_stride, pads, n_pads,
                            dilations, n_dil, group, auto_pad, auto_pad_len, g));
    if (bias && bias_len != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "bias holds %zu values for %d filters", bias_len, g.M);
    ZB_NEED_CTX(ctx);
    log_line("Running Conv [%d,%d,%d,%d] * [%d,%d,%d,%d]", g.N, g.C, g.H, g.W, g.M, g.Cg, g.KH, g.KW);
    if (ctx->tf32 && !is_device_ptr(w) && !(bias && is_device_ptr(bias)) && g.M <= 2048 && (long long)g.N * g.OH * g.OW >= 128) {
        // tensor-core path (2e-3 contract): weights blocked on the host, im2col gather + tcgen05 kind::tf32 GEMM
        TfGemmPrep prep;
        tf_gemm_prepare(w, g.M, g.C * g.KH * g.KW, (long long)g.C * g.KH * g.KW, 1, bias, prep, (long long)g.N * g.OH * g.OW, ctx->tf32 == 2);
        tf_conv_table(g, prep);
        Stager s(ctx);
        const int ix = s.in(x, numel(x_shape, 4) * 4), iy = s.out(y, numel(y_shape, 4) * 4);
        const int iw = s.in(prep.w_blk.data(), prep.w_blk.size() * 4), ib = s.in(prep.bias.data(), prep.bias.size() * 4);
        const int it = s.in(prep.ktab.data(), prep.ktab.size() * 4);
        const int ia = s.scratch(tf_gemm_a_bytes((size_t)g.N * g.OH * g.OW, prep));
        ZB_TRY(s.commit());
        ZB_TRY(run_conv_tf32(ctx, g, s.ptr<float>(ix), prep, s.ptr<float>(iw), s.ptr<float>(ib), s.ptr<int32_t>(it), s.ptr<float>(ia), FACT_NONE, 0.0f, s.ptr<float>(iy)));
        return s.finish();
    }
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, 4) * 4), iw = s.in(w, numel(w_shape, 4) * 4);
    const int ib = s.in(bias, (size_t)g.M * 4), iy = s.out(y, numel(y_shape, 4) * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_conv_f32(ctx, g, s.ptr<float>(ix), s.ptr<float>(iw), s.ptr<float>(ib), s.ptr<float>(iy)));
    return s.finish();
}

int32_t zant_b200_mat_mul_f32(zant_ctx* ctx, const float* a, const size_t* a_shape, size_t a_rank,
                              const float* b, const size_t* b_shape, size_t b_rank,
                              float* y, const size_t* y_shape, size_t y_rank) {
    ZB_NEED(a_shape, "a_shape"); ZB_NEED(b_shape, "b_shape"); ZB_NEED(y_shape, "y_shape");
    MatGeom g;
    ZB_TRY(matmul_check(a_shape, a_rank, b_shape, b_rank, y_shape, y_rank, g));
    ZB_NEED(a, "a"); ZB_NEED(b, "b"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    if (ctx->tf32 && !is_device_ptr(b) && g.N <= 2048 && g.M >= 128 && g.K <= 0x7fffffffULL && g.M <= 0x7fffffffULL) {
        TfGemmPrep prep;
        tf_gemm_prepare(b, (int)g.N, (int)g.K, 1, (long long)g.N, nullptr, prep, (long long)g.M, ctx->tf32 == 2);
        Stager s(ctx);
        const int ia = s.in(a, g.M * g.K * 4), iy = s.out(y, g.M * g.N * 4);
        const int iw = s.in(prep.w_blk.data(), prep.w_blk.size() * 4), ibz = s.in(prep.bias.data(), prep.bias.size() * 4);
        const int ik = s.scratch(tf_gemm_a_bytes(g.M, prep));
        ZB_TRY(s.commit());
        ZB_TRY(run_matmul_tf32(ctx, s.ptr<float>(ia), (long long)g.M, (int)g.K, (long long)g.K, 1, prep, s.ptr<float>(iw), s.ptr<float>(ibz), s.ptr<float>(ik),
                               FACT_NONE, 0.0f, s.ptr<float>(iy)));
        return s.finish();
    }
    Stager s(ctx);
    const int ia = s.in(a, g.M * g.K * 4), ib = s.in(b, g.K * g.N * 4), iy = s.out(y, g.M * g.N * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_matmul_f32(ctx, g, s.ptr<float>(ia), s.ptr<float>(ib), s.ptr<float>(iy)));
    return s.finish();
}

int32_t zant_b200_gemm_f32(zant_ctx* ctx, const float* a, const size_t* a_shape, size_t a_rank,
                           const float* b, const size_t* b_shape, size_t b_rank,
                           const float* c, const size_t* c_shape, size_t c_rank,
                           float alpha, float beta, int32_t trans_a, int32_t trans_b,
                           float* y, const size_t* y_shape, size_t y_rank) {
    ZB_NEED(a_shape, "a_shape"); ZB_NEED(b_shape, "b_shape");
    GemmGeom g;
    size_t auto_y[4];
    // the checks that do not involve the output run first, as in gemm() (op_gemm.zig:22-61)
    if (a_rank == 4 && b_rank == 4 && !y_shape) return fail(ZANT_E_NULL_POINTER, "y_shape is NULL");
    if (a_rank != 4 || b_rank != 4) { auto_y[0] = auto_y[1] = auto_y[2] = auto_y[3] = 0; y_shape = auto_y; y_rank = 4; }
    if (c && !c_shape) return fail(ZANT_E_NULL_POINTER, "c_shape is NULL");
    ZB_TRY(gemm_check(a_shape, a_rank, b_shape, b_rank, c_shape, c_rank, c != nullptr, trans_a != 0, trans_b != 0, beta,
                      y_shape, y_rank, g));
    ZB_NEED(a, "a"); ZB_NEED(b, "b"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ia = s.in(a, numel(a_shape, 4) * 4), ib = s.in(b, numel(b_shape, 4) * 4);
    const int ic = s.in(c, c ? numel(c_shape, 4) * 4 : 0), iy = s.out(y, numel(y_shape, 4) * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_gemm_f32(ctx, g, s.ptr<float>(ia), s.ptr<float>(ib), s.ptr<float>(ic), alpha, beta, trans_a != 0, trans_b != 0, s.ptr<float>(iy)));
    return s.finish();
}

int32_t zant_b200_gemm_lean_f32(zant_ctx* ctx, const float* a, const size_t* a_shape, size_t a_rank,
                                const float* b, const size_t* b_shape, size_t b_rank,
                                const float* c, const size_t* c_shape, size_t c_rank,
                                float alpha, float beta, int32_t trans_a, int32_t trans_b,
                                float* y, const size_t* y_shape, size_t y_rank) {
    ZB_NEED(a_shape, "a_shape"); ZB_NEED(b_shape, "b_shape"); ZB_NEED(y_shape, "y_shape");
    if (c && !c_shape) return fail(ZANT_E_NULL_POINTER, "c_shape is NULL");
    GemmGeom g;
    ZB_TRY(gemm_check_lean(a_shape, a_rank, b_shape, b_rank, c_shape, c_rank, c != nullptr, trans_a != 0, trans_b != 0, beta, y_shape, y_rank, g));
    ZB_NEED(a, "a"); ZB_NEED(b, "b"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ia = s.in(a, numel(a_shape, a_rank) * 4), ib = s.in(b, numel(b_shape, b_rank) * 4);
    const int ic = s.in(c, c ? numel(c_shape, c_rank) * 4 : 0), iy = s.out(y, numel(y_shape, y_rank) * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_gemm_f32(ctx, g, s.ptr<float>(ia), s.ptr<float>(ib), s.ptr<float>(ic), alpha, beta, trans_a != 0, trans_b != 0, s.ptr<float>(iy)));
    return s.finish();
}

int32_t zant_b200_maxpool_f32(zant_ctx* ctx, const float* x, const size_t* x_shape, size_t x_rank,
                              float* y, const size_t* y_shape, size_t y_rank,
                              const size_t* kernel_shape, size_t n_kernel, const size_t* strides, size_t n_strides,
                              const size_t* dilations, size_t n_dil, const size_t* pads, size_t n_pads, int32_t auto_pad) {
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(y_shape, "y_shape");
    PoolGeom g;
    ZB_TRY(pool_resolve(x_shape, x_rank, y_shape, y_rank, kernel_shape, n_kernel, strides, n_strides, dilations, n_dil, pads, n_pads, auto_pad, g));
    ZB_NEED(x, "x"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, 4) * 4), iy = s.out(y, numel(y_shape, 4) * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_maxpool<float>(ctx, g, s.ptr<float>(ix), s.ptr<float>(iy)));
    return s.finish();
}

}  // extern "C"

template <typename F>
static int32_t unary_entry(zant_ctx* ctx, const float* x, float* y, size_t n, F f, const char* name) {
    if (n) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, n * 4), iy = s.out(y, n * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_unary_f32(ctx, s.ptr<float>(ix), s.ptr<float>(iy), n, f, name));
    return s.finish();
}

extern "C" {

int32_t zant_b200_relu_f32(zant_ctx* ctx, const float* x, float* y, size_t n) { return unary_entry(ctx, x, y, n, ReluOp{}, "relu_f32"); }
int32_t zant_b200_leaky_relu_f32(zant_ctx* ctx, const float* x, float slope, float* y, size_t n) { return unary_entry(ctx, x, y, n, LeakyOp{slope}, "leaky_relu_f32"); }
int32_t zant_b200_clip_f32(zant_ctx* ctx, const float* x, float lo, float hi, float* y, size_t n) { return unary_entry(ctx, x, y, n, ClipOp{lo, hi}, "clip_f32"); }

int32_t zant_b200_sigmoid_f32(zant_ctx* ctx, const float* x, float* y, size_t n) { return unary_entry(ctx, x, y, n, SigmoidOp{}, "sigmoid_f32"); }
int32_t zant_b200_tanh_f32(zant_ctx* ctx, const float* x, float* y, size_t n) { return unary_entry(ctx, x, y, n, TanhOp{}, "tanh_f32"); }
int32_t zant_b200_ceil_f32(zant_ctx* ctx, const float* x, float* y, size_t n) { return unary_entry(ctx, x, y, n, CeilOp{}, "ceil_f32"); }

int32_t zant_b200_softmax_f32(zant_ctx* ctx, const float* x, float* y, size_t rows, size_t cols) {
    const size_t n = rows * cols;
    if (n) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, n * 4), iy = s.out(y, n * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_softmax_f32(ctx, s.ptr<float>(ix), s.ptr<float>(iy), rows, cols));
    return s.finish();
}

static int32_t binary_entry(zant_ctx* ctx, const float* a, size_t n_a, const float* b, size_t n_b, float* y, bool divide) {
    if (n_a != n_b) return fail(ZANT_E_MISMATCHED_SHAPE, "operands hold %zu and %zu elements", n_a, n_b);
    if (n_a) { ZB_NEED(a, "a"); ZB_NEED(b, "b"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ia = s.in(a, n_a * 4), ib = s.in(b, n_b * 4), iy = s.out(y, n_a * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_binary_same_f32(ctx, s.ptr<float>(ia), s.ptr<float>(ib), s.ptr<float>(iy), n_a, divide));
    return s.finish();
}
int32_t zant_b200_mul_f32(zant_ctx* ctx, const float* a, size_t n_a, const float* b, size_t n_b, float* y) { return binary_entry(ctx, a, n_a, b, n_b, y, false); }
int32_t zant_b200_div_f32(zant_ctx* ctx, const float* a, size_t n_a, const float* b, size_t n_b, float* y) { return binary_entry(ctx, a, n_a, b, n_b, y, true); }

int32_t zant_b200_sum_tensors_f32(zant_ctx* ctx, const float* a, const size_t* a_shape, size_t a_rank,
                                  const float* b, const size_t* b_shape, size_t b_rank,
                                  float* y, const size_t* y_shape, size_t y_rank) {
    ZB_NEED(a_shape, "a_shape"); ZB_NEED(b_shape, "b_shape"); ZB_NEED(y_shape, "y_shape");
    BcastGeom g;
    ZB_TRY(bcast_resolve(a_shape, a_rank, b_shape, b_rank, y_shape, y_rank, g));
    ZB_NEED(a, "a"); ZB_NEED(b, "b"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ia = s.in(a, numel(a_shape, a_rank) * 4), ib = s.in(b, numel(b_shape, b_rank) * 4), iy = s.out(y, g.total * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_add_f32(ctx, g, s.ptr<float>(ia), s.ptr<float>(ib), s.ptr<float>(iy)));
    return s.finish();
}

int32_t zant_b200_sum_tensor_list_f32(zant_ctx* ctx, const float* const* tensors, size_t n_tensors, float* y, size_t n) {
    if (n_tensors == 0) return fail(ZANT_E_EMPTY_TENSOR_LIST, "empty tensor list");
    ZB_NEED(tensors, "tensors"); ZB_NEED(y, "y");
    for (size_t t = 0; t < n_tensors; ++t) ZB_NEED(tensors[t], "tensors[i]");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    std::vector<int> idx(n_tensors);
    for (size_t t = 0; t < n_tensors; ++t) idx[t] = s.in(tensors[t], n * 4);
    const int iy = s.out(y, n * 4);
    ZB_TRY(s.commit());
    std::vector<const float*> dev(n_tensors);
    for (size_t t = 0; t < n_tensors; ++t) dev[t] = s.ptr<float>(idx[t]);
    ZB_TRY(run_sum_list_f32(ctx, dev.data(), n_tensors, s.ptr<float>(iy), n));
    return s.finish();
}

int32_t zant_b200_concatenate(zant_ctx* ctx, int32_t dtype, const void* const* tensors, const size_t* const* shapes,
                              const size_t* ranks, size_t n_tensors, int64_t axis, void* y, const size_t* y_shape, size_t y_rank) {
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    if (n_tensors) { ZB_NEED(shapes, "shapes"); ZB_NEED(ranks, "ranks"); }
    ConcatGeom g;
    size_t os[8];
    ZB_TRY(concat_resolve(shapes, ranks, n_tensors, axis, os, g));
    ZB_NEED(y_shape, "y_shape");
    if (y_rank != g.rank) return fail(ZANT_E_MISMATCHED_RANK, "output rank %zu != %zu", y_rank, g.rank);
    for (size_t d = 0; d < g.rank; ++d)
        if (y_shape[d] != os[d]) return fail(ZANT_E_INDEX_OUT_OF_BOUNDS, "output dim %zu is %zu, expected %zu", d, y_shape[d], os[d]);
    ZB_NEED(tensors, "tensors"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    const size_t esz = dtype_size(dtype);
    Stager s(ctx);
    std::vector<int> idx(n_tensors);
    for (size_t t = 0; t < n_tensors; ++t) idx[t] = s.in(tensors[t], g.num_slices * g.axis_dim[t] * g.slice * esz);
    const int iy = s.out(y, numel(os, g.rank) * esz);
    ZB_TRY(s.commit());
    std::vector<const void*> dev(n_tensors);
    for (size_t t = 0; t < n_tensors; ++t) dev[t] = s.ptr<char>(idx[t]);
    ZB_TRY(run_concat(ctx, g, esz, dev.data(), s.ptr<char>(iy)));
    return s.finish();
}

int32_t zant_b200_unsqueeze_output_shape(const size_t* x_shape, size_t x_rank, const int64_t* axes, size_t n_axes, size_t* out_shape) {
    if (x_rank) ZB_NEED(x_shape, "x_shape");
    if (n_axes) ZB_NEED(axes, "axes");
    ZB_NEED(out_shape, "out_shape");
    const size_t orank = x_rank + n_axes;
    if (orank > 16) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "output rank %zu", orank);
    bool is_new[16] = {false};
    for (size_t i = 0; i < n_axes; ++i) {
        long long a = axes[i];
        if (a < 0) a += (long long)orank;
        if (a < 0 || a >= (long long)orank) return fail(ZANT_E_AXIS_OUT_OF_BOUNDS, "axis %lld for output rank %zu", (long long)axes[i], orank);
        if (is_new[a]) return fail(ZANT_E_DUPLICATE_AXIS, "axis %lld given twice", (long long)axes[i]);
        is_new[a] = true;
    }
    size_t k = 0;
    for (size_t i = 0; i < orank; ++i) out_shape[i] = is_new[i] ? 1 : x_shape[k++];
    return ZANT_OK;
}

int32_t zant_b200_unsqueeze(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                            const int64_t* axes, size_t n_axes, void* y, const size_t* y_shape, size_t y_rank) {
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    size_t os[16];
    ZB_TRY(zant_b200_unsqueeze_output_shape(x_shape, x_rank, axes, n_axes, os));
    ZB_NEED(y_shape, "y_shape");
    if (y_rank != x_rank + n_axes) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output rank %zu, expected %zu", y_rank, x_rank + n_axes);
    for (size_t d = 0; d < y_rank; ++d)
        if (y_shape[d] != os[d]) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output dim %zu is %zu, expected %zu", d, y_shape[d], os[d]);
    const size_t bytes = numel(x_shape, x_rank) * dtype_size(dtype);
    if (bytes) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, bytes), iy = s.out(y, bytes);
    ZB_TRY(s.commit());
    ZB_TRY(run_copy2d(ctx, s.ptr<char>(ix), bytes, s.ptr<char>(iy), bytes, bytes, 1));
    return s.finish();
}

int32_t zant_b200_shape_onnx(const size_t* x_shape, size_t x_rank, int32_t has_start, int64_t start, int32_t has_end, int64_t end,
                             int64_t* out, size_t* out_len) {
    ZB_NEED(out_len, "out_len");
    if (x_rank == 0) { *out_len = 0; return ZANT_OK; }
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(out, "out");
    const long long r = (long long)x_rank;
    long long s0 = has_start ? start : 0; if (s0 < 0) s0 += r;
    long long e0 = has_end ? end : r; if (e0 < 0) e0 += r;
    // length as get_shape_output_shape counts it, values as lean_shape_onnx reads them (start clamped to rank - 1)
    const long long s_len = std::max(0LL, std::min(s0, r)), e_len = std::max(s_len, std::min(e0, r));
    const long long s_val = std::max(0LL, std::min(s0, r - 1)), e_val = std::max(s_val, std::min(e0, r));
    *out_len = (size_t)std::max(0LL, e_len - s_len);
    if ((size_t)std::max(0LL, e_val - s_val) != *out_len) return fail(ZANT_E_MISMATCHED_SHAPE, "shape_onnx: the reference's two clamps disagree (ShapeMismatch)");
    for (size_t i = 0; i < *out_len; ++i) out[i] = (int64_t)x_shape[(size_t)s_val + i];
    return ZANT_OK;
}

int32_t zant_b200_transpose_onnx(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                                 const size_t* perm, size_t n_perm, void* y, const size_t* y_shape, size_t y_rank) {
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    if (x_rank) { ZB_NEED(x_shape, "x_shape"); ZB_NEED(y_shape, "y_shape"); }
    StridedMap m;
    ZB_TRY(transpose_resolve(x_shape, x_rank, perm, n_perm, y_shape, y_rank, m));
    if (m.total) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    const size_t esz = dtype_size(dtype);
    Stager s(ctx);
    const int ix = s.in(x, m.total * esz), iy = s.out(y, m.total * esz);
    ZB_TRY(s.commit());
    ZB_TRY(run_strided_copy(ctx, esz, s.ptr<char>(ix), s.ptr<char>(iy), m));
    return s.finish();
}

int32_t zant_b200_slice_output_shape(const size_t* x_shape, size_t x_rank, const int64_t* starts, const int64_t* ends, size_t n,
                                     const int64_t* axes, const int64_t* steps, size_t* out_shape) {
    if (x_rank) { ZB_NEED(x_shape, "x_shape"); ZB_NEED(out_shape, "out_shape"); }
    if (n) { ZB_NEED(starts, "starts"); ZB_NEED(ends, "ends"); }
    return slice_resolve(x_shape, x_rank, starts, ends, n, axes, steps, out_shape, nullptr, true);
}

int32_t zant_b200_slice_lean_dims(const size_t* x_shape, size_t x_rank, const int64_t* starts, const int64_t* ends, size_t n,
                                  const int64_t* axes, const int64_t* steps, size_t* out_shape) {
    if (x_rank) { ZB_NEED(x_shape, "x_shape"); ZB_NEED(out_shape, "out_shape"); }
    if (n) { ZB_NEED(starts, "starts"); ZB_NEED(ends, "ends"); }
    return slice_resolve(x_shape, x_rank, starts, ends, n, axes, steps, out_shape, nullptr, false);
}

int32_t zant_b200_slice_onnx(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                             const int64_t* starts, const int64_t* ends, size_t n, const int64_t* axes, const int64_t* steps,
                             void* y, const size_t* y_shape, size_t y_rank) {
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    if (x_rank) { ZB_NEED(x_shape, "x_shape"); ZB_NEED(y_shape, "y_shape"); }
    if (n) { ZB_NEED(starts, "starts"); ZB_NEED(ends, "ends"); }
    StridedMap m;
    size_t od[8];
    ZB_TRY(slice_resolve(x_shape, x_rank, starts, ends, n, axes, steps, od, &m));
    if (y_rank != x_rank) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output rank %zu, input rank %zu", y_rank, x_rank);
    for (size_t d = 0; d < x_rank; ++d)
        if (y_shape[d] != od[d]) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output dim %zu is %zu, expected %zu", d, y_shape[d], od[d]);
    if (m.total) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    const size_t esz = dtype_size(dtype);
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, x_rank) * esz), iy = s.out(y, m.total * esz);
    ZB_TRY(s.commit());
    ZB_TRY(run_strided_copy(ctx, esz, s.ptr<char>(ix), s.ptr<char>(iy), m));
    return s.finish();
}

int32_t zant_b200_gather(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                         const size_t* indices, const size_t* idx_shape, size_t idx_rank, int64_t axis,
                         void* y, const size_t* y_shape, size_t y_rank) {
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    if (x_rank) ZB_NEED(x_shape, "x_shape");
    if (idx_rank) ZB_NEED(idx_shape, "idx_shape");
    ZB_NEED(y_shape, "y_shape");
    size_t n_idx = 1;
    for (size_t i = 0; i < idx_rank; ++i) n_idx *= idx_shape[i];
    if (n_idx) ZB_NEED(indices, "indices");
    if (is_device_ptr(indices)) return fail(ZANT_E_INVALID_INPUT, "gather indices must be a host array");
    GatherGeom g;
    ZB_TRY(gather_resolve(x_shape, x_rank, indices, idx_shape, idx_rank, axis, y_shape, y_rank, g));
    if (g.axis_dim > 0x7fffffffULL) return fail(ZANT_E_TOO_LARGE, "gather axis of %zu entries", g.axis_dim);
    const size_t total = g.outer * g.n_idx * g.inner;
    if (total) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    std::vector<int32_t> idx32(g.n_idx);
    for (size_t i = 0; i < g.n_idx; ++i) idx32[i] = (int32_t)indices[i];
    const size_t esz = dtype_size(dtype);
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, x_rank) * esz), ii = s.in(idx32.data(), idx32.size() * 4), iy = s.out(y, total * esz);
    ZB_TRY(s.commit());
    ZB_TRY(run_gather(ctx, esz, s.ptr<char>(ix), s.ptr<int32_t>(ii), s.ptr<char>(iy), g));
    return s.finish();
}

int32_t zant_b200_resize(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t rank,
                         const char* mode, size_t mode_len, const float* scales, size_t n_scales,
                         const size_t* sizes, size_t n_sizes, const char* coord_mode, size_t coord_mode_len,
                         void* y, const size_t* y_shape, size_t y_rank) {
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    ZB_NEED(x_shape, "x_shape");
    if (rank == 0 || rank > 8) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "rank %zu", rank);
    size_t os[8];
    ZB_TRY(resize_output_shape(x_shape, rank, scales, n_scales, sizes, n_sizes, os));
    if (!bytes_eq(mode, mode_len, "nearest")) {
        if (bytes_eq(mode, mode_len, "linear") || bytes_eq(mode, mode_len, "cubic"))
            return fail(ZANT_E_UNSUPPORTED, "Resize mode linear/cubic is not implemented by this back end");
        return fail(ZANT_E_UNSUPPORTED_MODE, "unknown Resize mode");
    }
    ZB_NEED(y_shape, "y_shape");
    if (y_rank != rank) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output rank");
    for (size_t d = 0; d < rank; ++d) if (y_shape[d] != os[d]) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output dim %zu is %zu, expected %zu", d, y_shape[d], os[d]);
    for (size_t d = 0; d < rank; ++d) if (x_shape[d] == 0) return fail(ZANT_E_EMPTY_TENSOR, "empty input");
    ZB_NEED(x, "x"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    std::vector<int32_t> table, axis_offset;
    resize_index_table(x_shape, os, rank, coord_mode_code(coord_mode, coord_mode_len), table, axis_offset);
    const size_t esz = dtype_size(dtype);
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, rank) * esz), iy = s.out(y, numel(os, rank) * esz);
    const int it = s.in(table.data(), std::max<size_t>(table.size(), 1) * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_resize(ctx, esz, s.ptr<char>(ix), s.ptr<char>(iy), s.ptr<int32_t>(it), x_shape, os, rank, axis_offset));
    return s.finish();
}

int32_t zant_b200_reduce_mean_f32(zant_ctx* ctx, const float* x, const size_t* x_shape, size_t x_rank,
                                  float* y, const size_t* y_shape, size_t y_rank,
                                  const int64_t* axes, size_t n_axes, int32_t keepdims, int32_t noop_with_empty_axes) {
    (void)keepdims;
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(y_shape, "y_shape");
    ReduceGeom g;
    ZB_TRY(reduce_resolve(x_shape, x_rank, y_shape, y_rank, axes, n_axes, noop_with_empty_axes != 0, g));
    ZB_NEED(x, "x"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, g.total * 4), iy = s.out(y, g.out_total * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_reduce_mean_f32(ctx, g, s.ptr<float>(ix), s.ptr<float>(iy)));
    return s.finish();
}

int32_t zant_b200_reshape(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                          const size_t* new_shape, size_t new_rank, void* y, size_t* y_shape_out) {
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(new_shape, "new_shape"); ZB_NEED(y_shape_out, "y_shape_out");
    if (new_rank > 16) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "rank %zu", new_rank);
    size_t out[16];
    ZB_TRY(reshape_resolve(x_shape, x_rank, new_shape, new_rank, out));
    for (size_t i = 0; i < new_rank; ++i) y_shape_out[i] = out[i];
    const size_t bytes = numel(x_shape, x_rank) * dtype_size(dtype);
    if (bytes == 0) return ZANT_OK;
    ZB_NEED(x, "x"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    // The reference copies (lib_shape_math.zig:1208); cudaMemcpyAsync picks the direction itself.
    ZB_CUDA(cudaMemcpyAsync(y, x, bytes, cudaMemcpyDefault, ctx->stream));
    if (!is_device_ptr(y) || !is_device_ptr(x)) ZB_CUDA(cudaStreamSynchronize(ctx->stream));
    return ZANT_OK;
}

// ------------------------------------------------------------------------------------ quantized operators
static bool q8_dtype(int32_t dt) { return dt == ZANT_I8 || dt == ZANT_U8; }

int32_t zant_b200_quantize_linear(zant_ctx* ctx, const float* x, size_t n, float scale, int32_t zero_point, int32_t out_dtype, void* y) {
    if (!q8_dtype(out_dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QuantizeLinear output must be int8 or uint8");
    if (n) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, n * 4), iy = s.out(y, n);
    ZB_TRY(s.commit());
    ZB_TRY(run_quantize(ctx, s.ptr<float>(ix), s.ptr<char>(iy), n, scale, zero_point, out_dtype));
    return s.finish();
}

int32_t zant_b200_dequantize_linear(zant_ctx* ctx, int32_t in_dtype, const void* q, size_t n, float scale, int32_t zero_point, float* y) {
    if (!q8_dtype(in_dtype) && in_dtype != ZANT_I32) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "DequantizeLinear input must be int8, uint8 or int32");
    if (n) { ZB_NEED(q, "q"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int iq = s.in(q, n * dtype_size(in_dtype)), iy = s.out(y, n * 4);
    ZB_TRY(s.commit());
    ZB_TRY(run_dequantize(ctx, in_dtype, s.ptr<char>(iq), s.ptr<float>(iy), n, scale, zero_point));
    return s.finish();
}

int32_t zant_b200_qlinearconv_nhwc(zant_ctx* ctx, int32_t x_dtype, const void* x, const size_t* x_shape, size_t x_rank,
                                   float x_scale, int32_t x_zp, const int8_t* w, const size_t* w_shape, size_t w_rank,
                                   const float* w_scale, const int32_t* w_zp, size_t n_w_scale, float y_scale, int32_t y_zp,
                                   const int32_t* bias, size_t bias_len, int32_t y_dtype, void* y, const size_t* y_shape, size_t y_rank,
                                   const size_t* stride, size_t n_stride, const size_t* pads, size_t n_pads,
                                   const size_t* dilations, size_t n_dil, size_t group, int32_t auto_pad, int32_t activation) {
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(w_shape, "w_shape"); ZB_NEED(y_shape, "y_shape");
    if (!q8_dtype(x_dtype) || !q8_dtype(y_dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearConv tensors must be int8 or uint8");
    ZB_TRY(check_zero_point(x_dtype, x_zp, "QLinearConv x"));
    if (x_rank != 4 || y_rank != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "channels-last QLinearConv takes rank-4 tensors");
    // the geometry is that of the NCHW operator on the permuted shapes
    const size_t xs[4] = {x_shape[0], x_shape[3], x_shape[1], x_shape[2]}, ys[4] = {y_shape[0], y_shape[3], y_shape[1], y_shape[2]};
    ConvGeom g;
    ZB_TRY(conv_resolve_onnx(xs, 4, w_shape, w_rank, ys, 4, stride, n_stride, pads, n_pads, dilations, n_dil, group, auto_pad, g));
    ZB_NEED(w_scale, "w_scale");
    if (n_w_scale != 1 && n_w_scale != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "w_scale holds %zu values for %d filters", n_w_scale, g.M);
    if (bias && bias_len != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "bias holds %zu values for %d filters", bias_len, g.M);
    if (activation < ZANT_QACT_NONE || activation > ZANT_QACT_RELU6) return fail(ZANT_E_INVALID_INPUT, "activation %d", activation);
    ZB_NEED(x, "x"); ZB_NEED(w, "w"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    if (is_device_ptr(w) || (bias && is_device_ptr(bias))) return fail(ZANT_E_UNSUPPORTED, "channels-last QLinearConv takes weights and bias from host memory");
    if ((is_device_ptr(x) && !tc_conv_ptr_ok(x)) || (is_device_ptr(y) && !tc_conv_ptr_ok(y))) return fail(ZANT_E_INVALID_INPUT, "channels-last QLinearConv buffers must be 16-byte aligned");
    std::vector<float> mult;
    requant_multipliers(x_scale, w_scale, n_w_scale, y_scale, (size_t)g.M, mult);
    bool wz_zero = true;
    if (w_zp) for (size_t i = 0; i < n_w_scale; ++i) wz_zero = wz_zero && w_zp[i] == 0;
    TcConvPlan tcp;
    if (!tc_conv_nhwc_plan(g, wz_zero, x_zp, tcp)) return fail(ZANT_E_UNSUPPORTED, "shape not taken by the channels-last QLinearConv kernel");
    std::vector<int8_t> w_blk; std::vector<float> mp; std::vector<int32_t> bp;
    tc_conv_nhwc_prepare(tcp, w, mult.data(), bias, x_zp, w_blk, mp, bp);
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, 4)), iy = s.out(y, numel(y_shape, 4));
    const int iw = s.in(w_blk.data(), w_blk.size()), im = s.in(mp.data(), mp.size() * 4), ib = s.in(bp.data(), bp.size() * 4);
    ZB_TRY(s.commit());
    ZB_TRY(tc_conv_nhwc_run(ctx, tcp, s.ptr<char>(ix), x_dtype == ZANT_U8, s.ptr<int8_t>(iw), s.ptr<float>(im), s.ptr<int32_t>(ib),
                            s.ptr<char>(iy), y_dtype == ZANT_U8, Requant{y_scale, y_zp, activation}, tc_conv_max_product(mp, bp, (long long)g.Cg * g.KH * g.KW)));
    return s.finish();
}

int32_t zant_b200_qlinearconv(zant_ctx* ctx, int32_t x_dtype, const void* x, const size_t* x_shape, size_t x_rank,
                              float x_scale, int32_t x_zp, const int8_t* w, const size_t* w_shape, size_t w_rank,
                              const float* w_scale, const int32_t* w_zp, size_t n_w_scale, float y_scale, int32_t y_zp,
                              const int32_t* bias, size_t bias_len, int32_t y_dtype, void* y, const size_t* y_shape, size_t y_rank,
                              const size_t* stride, size_t n_stride, const size_t* pads, size_t n_pads,
                              const size_t* dilations, size_t n_dil, size_t group, int32_t auto_pad, int32_t activation) {
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(w_shape, "w_shape"); ZB_NEED(y_shape, "y_shape");
    if (!q8_dtype(x_dtype) || !q8_dtype(y_dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearConv tensors must be int8 or uint8");
    ZB_TRY(check_zero_point(x_dtype, x_zp, "QLinearConv x"));
    ConvGeom g;
    ZB_TRY(conv_resolve_onnx(x_shape, x_rank, w_shape, w_rank, y_shape, y_rank, stride, n_stride, pads, n_pads, dilations, n_dil, group, auto_pad, g));
    ZB_NEED(w_scale, "w_scale");
    if (n_w_scale != 1 && n_w_scale != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "w_scale holds %zu values for %d filters", n_w_scale, g.M);
    if (bias && bias_len != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "bias holds %zu values for %d filters", bias_len, g.M);
    if (activation < ZANT_QACT_NONE || activation > ZANT_QACT_RELU6) return fail(ZANT_E_INVALID_INPUT, "activation %d", activation);
    ZB_NEED(x, "x"); ZB_NEED(w, "w"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    std::vector<float> mult;
    requant_multipliers(x_scale, w_scale, n_w_scale, y_scale, (size_t)g.M, mult);
    std::vector<int32_t> wz((size_t)g.M, 0);
    if (w_zp) for (int m = 0; m < g.M; ++m) wz[m] = w_zp[n_w_scale == 1 ? 0 : m];
    bool wz_zero = true;
    for (int32_t v : wz) wz_zero = wz_zero && v == 0;
    const bool host_consts = !is_device_ptr(w) && !(bias && is_device_ptr(bias));
    PwConvPlan pwp;
    if (host_consts && (!is_device_ptr(x) || pw_conv_ptr_ok(x, nullptr)) && (!is_device_ptr(y) || pw_conv_ptr_ok(nullptr, y)) &&
        (pw_stem_plan(g, wz_zero, x_zp, ctx->sm_count, pwp) || pw_conv_plan(g, wz_zero, ctx->sm_count, pwp))) {
        // 1x1: filters on the accumulator lanes, activations straight from NCHW as the MN-major operand; 3x3 stems: the same
        // kernel on patches written in shared memory
        std::vector<int8_t> w_blk; std::vector<int32_t> bf;
        pw_conv_prepare(pwp, w, bias, x_zp, w_blk, bf);
        bool finite = true;
        for (float f : mult) finite = finite && std::isfinite(f);
        std::vector<int32_t> caps;
        const bool capped = finite && y_dtype == ZANT_I8 && y_zp == 0 && requant_relu_caps(mult.data(), mult.size(), activation, lean_six(y_scale), caps);
        Stager s(ctx);
        const int ix = s.in(x, numel(x_shape, 4)), iy = s.out(y, numel(y_shape, 4));
        const int iw = s.in(w_blk.data(), w_blk.size()), im = s.in(mult.data(), mult.size() * 4), ib = s.in(bf.data(), bf.size() * 4);
        const int ic = capped ? s.in(caps.data(), caps.size() * 4) : -1;
        ZB_TRY(s.commit());
        ZB_TRY(pw_conv_run(ctx, pwp, s.ptr<char>(ix), x_dtype == ZANT_U8, s.ptr<int8_t>(iw), s.ptr<float>(im), s.ptr<int32_t>(ib),
                           s.ptr<char>(iy), y_dtype == ZANT_U8, Requant{y_scale, y_zp, activation}, finite, capped ? s.ptr<int32_t>(ic) : nullptr));
        return s.finish();
    }
    if (host_consts && qconv_smallc_eligible(g, wz_zero) && (!is_device_ptr(x) || qconv_smallc_ptr_ok(x))) {
        // 3x3 on at most four input channels (network stems): warp-level MMAs with the filters as rows
        std::vector<uint32_t> wfrag; std::vector<int32_t> bf;
        qconv_smallc_prepare(g, w, bias, x_zp, wfrag, bf);
        Stager s(ctx);
        const int ix = s.in(x, numel(x_shape, 4)), iy = s.out(y, numel(y_shape, 4));
        const int iw = s.in(wfrag.data(), wfrag.size() * 4), im = s.in(mult.data(), mult.size() * 4), ib = s.in(bf.data(), bf.size() * 4);
        ZB_TRY(s.commit());
        ZB_TRY(run_qconv_smallc(ctx, g, s.ptr<char>(ix), x_dtype == ZANT_U8, x_zp, s.ptr<uint32_t>(iw), s.ptr<float>(im), s.ptr<int32_t>(ib),
                                s.ptr<char>(iy), y_dtype == ZANT_U8, Requant{y_scale, y_zp, activation}, tc_conv_max_product(mult, bf, (long long)g.C * 9)));
        return s.finish();
    }
    TcConvPlan tcp;
    if (host_consts && (long long)g.N * g.OH * g.OW >= 256 && (!is_device_ptr(x) || tc_conv_ptr_ok(x)) && tc_conv_plan(g, wz_zero, tcp)) {
        // implicit GEMM straight from NCHW (stride 1): no im2col matrix
        std::vector<int8_t> w_blk; std::vector<float> mp; std::vector<int32_t> bp;
        tc_conv_prepare(tcp, w, mult.data(), bias, x_zp, w_blk, mp, bp);
        Stager s(ctx);
        const int ix = s.in(x, numel(x_shape, 4)), iy = s.out(y, numel(y_shape, 4));
        const int iw = s.in(w_blk.data(), w_blk.size()), im = s.in(mp.data(), mp.size() * 4), ib = s.in(bp.data(), bp.size() * 4);
        ZB_TRY(s.commit());
        ZB_TRY(tc_conv_run(ctx, tcp, s.ptr<char>(ix), x_dtype == ZANT_U8, x_zp, s.ptr<int8_t>(iw), s.ptr<float>(im), s.ptr<int32_t>(ib),
                           s.ptr<char>(iy), y_dtype == ZANT_U8, Requant{y_scale, y_zp, activation}, tc_conv_max_product(mp, bp, (long long)g.Cg * g.KH * g.KW)));
        return s.finish();
    }
    if (host_consts && qdwconv_eligible(g, wz_zero) && (!is_device_ptr(x) || qdwconv_ptr_ok(x)) && (!is_device_ptr(y) || qdwconv_ptr_ok(y))) {
        // depthwise 3x3: one HBM-bound pass
        std::vector<uint32_t> wrow; std::vector<int32_t> bf;
        qdwconv_prepare(g, w, bias, x_zp, wrow, bf);
        bool finite = true;
        for (float f : mult) finite = finite && std::isfinite(f);
        std::vector<int32_t> caps;
        const bool capped = finite && y_dtype == ZANT_I8 && y_zp == 0 && requant_relu_caps(mult.data(), mult.size(), activation, lean_six(y_scale), caps);
        Stager s(ctx);
        const int ix = s.in(x, numel(x_shape, 4)), iy = s.out(y, numel(y_shape, 4));
        const int iw = s.in(wrow.data(), wrow.size() * 4), im = s.in(mult.data(), mult.size() * 4), ib = s.in(bf.data(), bf.size() * 4);
        const int ic = capped ? s.in(caps.data(), caps.size() * 4) : -1;
        ZB_TRY(s.commit());
        ZB_TRY(run_qdwconv(ctx, g, s.ptr<char>(ix), x_dtype == ZANT_U8, x_zp, s.ptr<uint32_t>(iw), s.ptr<float>(im), s.ptr<int32_t>(ib),
                           s.ptr<char>(iy), y_dtype == ZANT_U8, Requant{y_scale, y_zp, activation}, finite, capped ? s.ptr<int32_t>(ic) : nullptr));
        return s.finish();
    }
    if (qconv_tc_eligible(g, wz_zero) && host_consts) {
        // tensor-core path: im2col into the GEMM-blocked layout, tcgen05 GEMM, NCHW requantised store
        QGemmPrep prep;
        qconv_gemm_prepare(g, w, mult.data(), bias, x_zp, prep);
        Stager s(ctx);
        const int ix = s.in(x, numel(x_shape, 4)), iy = s.out(y, numel(y_shape, 4));
        const int iw = s.in(prep.w_blk.data(), prep.w_blk.size()), im = s.in(prep.mult.data(), prep.mult.size() * 4);
        const int ib = s.in(prep.bias.data(), prep.bias.size() * 4);
        const int ia = s.scratch(qgemm_a_bytes((size_t)g.N * g.OH * g.OW, prep));
        ZB_TRY(s.commit());
        ZB_TRY(run_qconv_tc(ctx, g, s.ptr<char>(ix), x_dtype == ZANT_U8, x_zp, prep, s.ptr<int8_t>(iw), s.ptr<float>(im), s.ptr<int32_t>(ib),
                            s.ptr<uint8_t>(ia), s.ptr<char>(iy), y_dtype == ZANT_U8, Requant{y_scale, y_zp, activation}));
        return s.finish();
    }
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, 4)), iw = s.in(w, numel(w_shape, 4)), iy = s.out(y, numel(y_shape, 4));
    const int im = s.in(mult.data(), mult.size() * 4), iz = s.in(wz.data(), wz.size() * 4), ib = s.in(bias, (size_t)g.M * 4);
    ZB_TRY(s.commit());
    QConvArgs p{};
    p.x = s.ptr<char>(ix); p.w = s.ptr<int8_t>(iw); p.y = s.ptr<char>(iy);
    p.mult = s.ptr<float>(im); p.w_zp = s.ptr<int32_t>(iz); p.bias = s.ptr<int32_t>(ib);
    p.x_zp = x_zp; p.rq = Requant{y_scale, y_zp, activation}; p.g = g;
    ZB_TRY(run_qconv_generic(ctx, p, x_dtype, y_dtype));
    return s.finish();
}

int32_t zant_b200_qlinearmatmul(zant_ctx* ctx, int32_t a_dtype, const void* a, const size_t* a_shape, size_t a_rank,
                                float a_scale, int32_t a_zp, const int8_t* b, const size_t* b_shape, size_t b_rank,
                                const float* b_scale, const int32_t* b_zp, size_t n_b_scale, float y_scale, int32_t y_zp,
                                const int32_t* bias, size_t bias_len, int32_t y_dtype, void* y, const size_t* y_shape, size_t y_rank,
                                int32_t activation) {
    ZB_NEED(a_shape, "a_shape"); ZB_NEED(b_shape, "b_shape"); ZB_NEED(y_shape, "y_shape");
    if (a_rank != 2 || b_rank != 2 || y_rank != 2) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearMatMul takes 2-D operands");
    if (!q8_dtype(a_dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "A must be int8 or uint8");
    ZB_TRY(check_zero_point(a_dtype, a_zp, "QLinearMatMul a"));
    if (!q8_dtype(y_dtype) && y_dtype != ZANT_I32) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "Y must be int8, uint8 or int32");
    const size_t M = a_shape[0], K = a_shape[1], N = b_shape[1];
    if (b_shape[0] != K) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "A cols %zu != B rows %zu", K, b_shape[0]);
    if (M * N == 0 || K == 0) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "empty operand");
    if (y_shape[0] != M || y_shape[1] != N) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "output is not [%zu,%zu]", M, N);
    ZB_NEED(b_scale, "b_scale");
    if (n_b_scale != 1 && n_b_scale != N) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "b_scale holds %zu values for %zu columns", n_b_scale, N);
    if (bias && bias_len != N) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "bias holds %zu values for %zu columns", bias_len, N);
    if (M > 0x7fffffffULL || N > 0x7fffffffULL || K > 0x7fffffffULL) return fail(ZANT_E_TOO_LARGE, "dims exceed int range");
    ZB_NEED(a, "a"); ZB_NEED(b, "b"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    std::vector<float> mult;
    requant_multipliers(a_scale, b_scale, n_b_scale, y_scale, N, mult);
    std::vector<int32_t> bz(N, 0);
    if (b_zp) for (size_t j = 0; j < N; ++j) bz[j] = b_zp[n_b_scale == 1 ? 0 : j];
    bool bz_zero = true;
    for (int32_t v : bz) bz_zero = bz_zero && v == 0;
    {
        ConvGeom g{};   // a matrix product is a 1x1 convolution over M "images" of one pixel
        g.N = (int)M; g.C = (int)K; g.H = g.W = 1; g.M = (int)N; g.Cg = (int)K; g.KH = g.KW = 1;
        g.sh = g.sw = g.dh = g.dw = 1; g.OH = g.OW = 1; g.G = 1;
        if (y_dtype != ZANT_I32 && qconv_tc_eligible(g, bz_zero) && !is_device_ptr(b) && !(bias && is_device_ptr(bias))) {
            std::vector<int8_t> bt(K * N);
            for (size_t k = 0; k < K; ++k) for (size_t j = 0; j < N; ++j) bt[j * K + k] = b[k * N + j];
            QGemmPrep prep;
            qgemm_prepare(bt.data(), (int)N, (int)K, mult.data(), bias, a_zp, prep);
            Stager s(ctx);
            const int ix = s.in(a, M * K), iy = s.out(y, M * N);
            const int iw = s.in(prep.w_blk.data(), prep.w_blk.size()), im = s.in(prep.mult.data(), prep.mult.size() * 4);
            const int ibb = s.in(prep.bias.data(), prep.bias.size() * 4);
            const int isc = s.scratch(qgemm_a_bytes(M, prep));
            ZB_TRY(s.commit());
            ZB_TRY(run_qconv_tc(ctx, g, s.ptr<char>(ix), a_dtype == ZANT_U8, a_zp, prep, s.ptr<int8_t>(iw), s.ptr<float>(im), s.ptr<int32_t>(ibb),
                                s.ptr<uint8_t>(isc), s.ptr<char>(iy), y_dtype == ZANT_U8, Requant{y_scale, y_zp, activation}));
            return s.finish();
        }
    }
    Stager s(ctx);
    const int ia = s.in(a, M * K), ib = s.in(b, K * N), iy = s.out(y, M * N * dtype_size(y_dtype));
    const int im = s.in(mult.data(), N * 4), iz = s.in(bz.data(), N * 4), ibias = s.in(bias, N * 4);
    ZB_TRY(s.commit());
    QMatArgs p{};
    p.a = s.ptr<char>(ia); p.b = s.ptr<int8_t>(ib); p.y = s.ptr<char>(iy);
    p.mult = s.ptr<float>(im); p.b_zp = s.ptr<int32_t>(iz); p.bias = s.ptr<int32_t>(ibias);
    p.a_zp = a_zp; p.rq = Requant{y_scale, y_zp, activation}; p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.y_i32 = y_dtype == ZANT_I32;
    ZB_TRY(run_qmatmul_generic(ctx, p, a_dtype, y_dtype));
    return s.finish();
}

int32_t zant_b200_qlinearadd(zant_ctx* ctx, int32_t dtype, const void* a, float a_scale, int32_t a_zp,
                             const void* b, float b_scale, int32_t b_zp, float y_scale, int32_t y_zp, void* y, size_t n,
                             int32_t activation) {
    if (!q8_dtype(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearAdd tensors must be int8 or uint8");
    if (n) { ZB_NEED(a, "a"); ZB_NEED(b, "b"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ia = s.in(a, n), ib = s.in(b, n), iy = s.out(y, n);
    ZB_TRY(s.commit());
    ZB_TRY(run_qadd(ctx, dtype, s.ptr<char>(ia), a_scale, a_zp, s.ptr<char>(ib), b_scale, b_zp, y_scale, y_zp, activation, s.ptr<char>(iy), n));
    return s.finish();
}

int32_t zant_b200_qlinear_global_avgpool(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                                         float x_scale, int32_t x_zp, float y_scale, int32_t y_zp, void* y) {
    if (!q8_dtype(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "tensors must be int8 or uint8");
    ZB_NEED(x_shape, "x_shape");
    if (x_rank != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "GlobalAveragePool needs a 4-D input");
    const size_t planes = x_shape[0] * x_shape[1], hw = x_shape[2] * x_shape[3];
    if (hw == 0 || hw > 0x7fffffffULL) return fail(ZANT_E_INVALID_DIMENSIONS, "H*W = %zu", hw);
    ZB_NEED(x, "x"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, planes * hw), iy = s.out(y, planes);
    ZB_TRY(s.commit());
    ZB_TRY(run_qgap(ctx, dtype, s.ptr<char>(ix), s.ptr<char>(iy), planes, (int)hw, x_scale, x_zp, y_scale, y_zp));
    return s.finish();
}

int32_t zant_b200_maxpool_q8(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                             void* y, const size_t* y_shape, size_t y_rank,
                             const size_t* kernel_shape, size_t n_kernel, const size_t* strides, size_t n_strides,
                             const size_t* dilations, size_t n_dil, const size_t* pads, size_t n_pads, int32_t auto_pad) {
    if (!q8_dtype(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "tensors must be int8 or uint8");
    ZB_NEED(x_shape, "x_shape"); ZB_NEED(y_shape, "y_shape");
    PoolGeom g;
    ZB_TRY(pool_resolve(x_shape, x_rank, y_shape, y_rank, kernel_shape, n_kernel, strides, n_strides, dilations, n_dil, pads, n_pads, auto_pad, g));
    ZB_NEED(x, "x"); ZB_NEED(y, "y");
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, numel(x_shape, 4)), iy = s.out(y, numel(y_shape, 4));
    ZB_TRY(s.commit());
    if (dtype == ZANT_U8) ZB_TRY(run_maxpool<uint8_t>(ctx, g, s.ptr<uint8_t>(ix), s.ptr<uint8_t>(iy)));
    else ZB_TRY(run_maxpool<int8_t>(ctx, g, s.ptr<int8_t>(ix), s.ptr<int8_t>(iy)));
    return s.finish();
}

int32_t zant_b200_lut_q8(zant_ctx* ctx, const void* x, const uint8_t lut[256], void* y, size_t n) {
    ZB_NEED(lut, "lut");
    if (n) { ZB_NEED(x, "x"); ZB_NEED(y, "y"); }
    ZB_NEED_CTX(ctx);
    Stager s(ctx);
    const int ix = s.in(x, n), iy = s.out(y, n), il = s.in(lut, 256);
    ZB_TRY(s.commit());
    ZB_TRY(run_lut(ctx, s.ptr<char>(ix), s.ptr<char>(iy), n, s.ptr<uint8_t>(il)));
    return s.finish();
}

}  // extern "C"
