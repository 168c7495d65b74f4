/*
 * zant_b200.h — C ABI of the B200 (sm_100a) backend for Z-Ant's TensorMath inference path.
 *
 * Every entry point replaces one function that Z-Ant's code generator emits calls to
 * (the name table is src/Core/Tensor/TensorMath/tensor_math_standard.zig in the Z-Ant tree);
 * the citation above each declaration names the function it stands in for.  Quantized entry
 * points have no counterpart in that tree (src/Core/Quantization/quantization.zig is empty):
 * they follow the ONNX operator definitions with the arithmetic order written in the comment.
 *
 * Conventions
 *   - Plain pointers and sizes only.  Shapes are `const size_t*` + rank, row-major, NCHW for
 *     4-D tensors (the layout Z-Ant's Tensor(T) uses, src/Core/Tensor/tensor.zig:25-31).
 *   - A data pointer may be a host pointer or a device pointer of the context's device; the
 *     library classifies it with cudaPointerGetAttributes.  Host buffers are staged through
 *     the context's device arena and the call returns after the result is back on the host;
 *     device buffers are used in place and the call is asynchronous on the context's stream.
 *   - Byte strings from Zig slices (auto_pad, modes) are (ptr,len) pairs, NOT NUL terminated.
 *   - Every function returns a zant_status: 0 on success, a negative code named after the Zig
 *     error the reference would have returned, or ZANT_E_CUDA* for device failures.  Nothing
 *     aborts the process.  There is no CPU fallback: without a usable device every compute
 *     entry point returns ZANT_E_CUDA_UNAVAILABLE.
 *   - A context is bound to one device and one stream and is not thread-safe; use one
 *     context per (thread, device).
 */
#ifndef ZANT_B200_H
#define ZANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------
 * Status codes.  Negative values mirror src/Utils/errorHandler.zig:36-84
 * (TensorMathError: -1..-14, TensorError: -33..-61); backend-specific codes start at -100.
 * ---------------------------------------------------------------------------------------- */
typedef enum zant_status {
    ZANT_OK = 0,
    /* TensorMathError */
    ZANT_E_INVALID_DIMENSIONS = -1,
    ZANT_E_MEM_ERROR = -2,
    ZANT_E_INPUT_TENSOR_DIFFERENT_SIZE = -3,
    ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE = -4,
    ZANT_E_INPUT_TENSORS_WRONG_SHAPE = -5,
    ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE = -6,
    ZANT_E_TOO_SMALL_OUTPUT_TYPE = -7,
    ZANT_E_INPUT_TENSOR_DIMENSION_MISMATCH = -8,
    ZANT_E_WRONG_STRIDE = -9,
    ZANT_E_INCOMPATIBLE_BROADCAST_SHAPES = -10,
    ZANT_E_EMPTY_TENSOR_LIST = -11,
    ZANT_E_DIVISION_ERROR = -12,
    ZANT_E_INVALID_PADDING = -13,
    ZANT_E_INVALID_AXES = -14,
    /* TensorError */
    ZANT_E_TENSOR_NOT_INITIALIZED = -33,
    ZANT_E_INPUT_ARRAY_WRONG_TYPE = -34,
    ZANT_E_INPUT_ARRAY_WRONG_SIZE = -35,
    ZANT_E_EMPTY_TENSOR = -36,
    ZANT_E_ZERO_SIZE_TENSOR = -37,
    ZANT_E_INVALID_SLICE_INDICES = -43,
    ZANT_E_INVALID_SLICE_STEP = -46,
    ZANT_E_AXIS_OUT_OF_BOUNDS = -49,
    ZANT_E_MISMATCHED_RANK = -50,
    ZANT_E_MISMATCHED_SHAPE = -51,
    ZANT_E_INDEX_OUT_OF_BOUNDS = -52,
    ZANT_E_INVALID_AXIS = -53,
    ZANT_E_DUPLICATE_AXIS = -54,
    ZANT_E_INVALID_INPUT = -55,
    ZANT_E_UNSUPPORTED_MODE = -56,
    ZANT_E_UNSUPPORTED_DIMENSION = -57,
    ZANT_E_INVALID_RANK = -59,
    ZANT_E_INVALID_PERMUTATION = -60,
    /* backend */
    ZANT_E_CUDA = -100,             /* a CUDA runtime call failed; see zant_b200_last_error() */
    ZANT_E_CUDA_UNAVAILABLE = -101, /* no usable sm_100 device / driver */
    ZANT_E_NULL_POINTER = -102,
    ZANT_E_UNSUPPORTED = -103,      /* valid ONNX, not implemented by this backend */
    ZANT_E_ARENA_EXHAUSTED = -104,
    ZANT_E_BAD_HANDLE = -105,
    ZANT_E_DEVICE_TIMEOUT = -106,   /* a bounded device-side wait gave up */
    ZANT_E_TOO_LARGE = -107
} zant_status;

typedef enum zant_dtype {
    ZANT_F32 = 0,
    ZANT_I8 = 1,
    ZANT_U8 = 2,
    ZANT_I32 = 3
} zant_dtype;

/* AutoPadType of src/Core/Tensor/TensorMath/op_pooling.zig:9-14 (same ordinal values). */
typedef enum zant_auto_pad {
    ZANT_PAD_NOTSET = 0,
    ZANT_PAD_SAME_UPPER = 1,
    ZANT_PAD_SAME_LOWER = 2,
    ZANT_PAD_VALID = 3
} zant_auto_pad;

/* Activation that a quantized producer may fuse into its epilogue. */
typedef enum zant_qact {
    ZANT_QACT_NONE = 0,
    ZANT_QACT_RELU = 1,  /* max(y, y_zp) */
    ZANT_QACT_RELU6 = 2  /* additionally min(y, sat(rne(6 / y_scale) + y_zp)) */
} zant_qact;

typedef struct zant_ctx zant_ctx;
typedef struct zant_plan zant_plan;

/* ------------------------------------------------------------------------------------------
 * Library, context, diagnostics
 * ---------------------------------------------------------------------------------------- */

/* Version string of this library ("zant-b200 x.y"). No reference counterpart. */
const char* zant_b200_version(void);

/* Name of a status code ("InvalidDimensions", ...), the Zig error name where one exists. */
const char* zant_b200_status_name(int32_t status);

/* Message of the last failure on the calling thread ("" if none). */
const char* zant_b200_last_error(void);

/* Number of visible CUDA devices (0 when the driver is absent). Never fails. */
int32_t zant_b200_device_count(void);

/* Replaces the generated library's setLogFunction / TensorMath's setLogFunctionC
 * (src/codeGen/skeleton.zig:90-100, src/Core/Tensor/TensorMath/op_convolution.zig:37-41):
 * installs a C callback that receives one NUL-terminated line per logged event. */
void zant_b200_set_log(void (*fn)(char* msg));

/* Creates a context on `device` with its own stream and a device staging arena of
 * `arena_bytes` (0 = default 256 MiB, grown on demand for host-pointer calls). */
int32_t zant_b200_ctx_create(int32_t device, size_t arena_bytes, zant_ctx** out);
int32_t zant_b200_ctx_destroy(zant_ctx* ctx);
/* Use a caller-owned cudaStream_t (passed as void*) instead of the context's own. */
int32_t zant_b200_ctx_set_stream(zant_ctx* ctx, void* cuda_stream);
/* Float precision of the contractions (Conv, MatMul, Gemm) issued through this context.  Off (the default, unless
 * the environment variable ZANT_B200_TF32 is set when the context is created): the exact FP32 kernels, which keep
 * the reference's order of operations (sequential fp32 accumulation, op_mat_mul.zig:132-148) and are bit-identical
 * to it.  1: tensor-core kernels (tcgen05 kind::tf32, operands rounded to TF32, fp32 accumulation), one MMA per K step;
 * the error of an output is about 3e-4 of the root sum of squares of its products: within 2e-3 of the output's scale,
 * |y - ref| <= 2e-3 * max|ref|, but not relative to outputs that are near-cancellations.  2: the
 * same kernels with every operand split into two TF32 parts (three MMAs per K step), which recovers about 21 bits of the
 * products: within |y - ref| <= 2e-3 * max(|ref|, 1e-2 * max|ref|) with a wide margin (in practice within the 1e-4 rule
 * of the FP32 path), at about half the speed of mode 1.  A plan takes the setting of its context when it is finalized;
 * zant_b200_conv_f32 and zant_b200_mat_mul_f32 take it at each call.  No reference counterpart. */
int32_t zant_b200_ctx_set_tf32(zant_ctx* ctx, int32_t enable);
int32_t zant_b200_ctx_get_tf32(zant_ctx* ctx);

/* Caps the staging arena that host-pointer calls grow on demand (0 = no cap, the default).  A call
 * whose host buffers and workspace need more returns ZANT_E_ARENA_EXHAUSTED and changes nothing;
 * device-pointer calls and plans (which own their arena) are not affected.  No reference
 * counterpart: the reference allocates temporaries from the process heap. */
int32_t zant_b200_ctx_set_arena_limit(zant_ctx* ctx, size_t max_bytes);
/* The stream kernels are launched on (a cudaStream_t as void*). */
void* zant_b200_ctx_stream(zant_ctx* ctx);
int32_t zant_b200_ctx_synchronize(zant_ctx* ctx);
/* Kernels launched by this context since creation (or since the last reset). */
uint64_t zant_b200_ctx_launch_count(zant_ctx* ctx);
void zant_b200_ctx_reset_launch_count(zant_ctx* ctx);

/* Attainable int8 tensor-core rate of the context's device in TOP/s: a resident-tile
 * tcgen05.mma kind::i8 loop (128x256x32 per instruction, `iters` x 2 instructions per SM, no
 * global traffic), best of four timed launches.  No reference counterpart; it is the
 * denominator of the roofline fractions reported for tensor-bound kernels. */
int32_t zant_b200_measure_int8_peak(zant_ctx* ctx, int32_t iters, double* tera_ops_per_s);

/* The same probe issued back to back for `seconds` (clamped to [0.05, 10]) and timed as one span: the rate the
 * tensor cores sustain under the power cap, the denominator for kernels timed inside a seconds-long loop. */
int32_t zant_b200_measure_int8_peak_sustained(zant_ctx* ctx, double seconds, double* tera_ops_per_s);

/* Failure-path self test (no reference counterpart).  Launches one CTA that allocates tensor
 * memory and waits, with the same bounded wait the tensor-core kernels use but a budget of
 * `budget_us` microseconds (clamped to [1, 100000]), on a barrier that nothing arrives on.  The
 * wait gives up, the kernel frees its tensor memory, records the time-out in the context's status
 * word and returns; nothing faults or hangs.  The launch itself returns ZANT_OK; the next
 * zant_b200_ctx_synchronize (or any call that waits for the stream) returns
 * ZANT_E_DEVICE_TIMEOUT once and clears the word, after which the context works as before. */
int32_t zant_b200_selftest_bounded_wait(zant_ctx* ctx, uint32_t budget_us);

/* Test hook (no reference counterpart): makes the `nth` next device allocation of this library
 * (1 = the very next one) fail as if the driver had answered cudaErrorMemoryAllocation, without
 * touching the driver; 0 disarms it.  Entry points that allocate (zant_b200_ctx_create, host-buffer
 * staging, zant_b200_plan_finalize) then return ZANT_E_MEM_ERROR, the reference's MemError
 * (src/Utils/errorHandler.zig:36-52), and leave their handles usable or destroyable. */
int32_t zant_b200_debug_fail_alloc(int32_t nth);

/* ------------------------------------------------------------------------------------------
 * Shape helpers (host only; usable without a GPU)
 * ---------------------------------------------------------------------------------------- */

/* Output shape of OnnxConv (op_convolution.zig:647-745; the generator's
 * get_convolution_output_shape :333-371 returns the same values). `group` 0 means "null". */
int32_t zant_b200_conv_output_shape(const size_t* x_shape, size_t x_rank,
                                    const size_t* w_shape, size_t w_rank,
                                    const size_t* stride, size_t n_stride,
                                    const size_t* pads, size_t n_pads,
                                    const size_t* dilations, size_t n_dil,
                                    const char* auto_pad, size_t auto_pad_len,
                                    size_t out_shape[4]);

/* get_pooling_output_shape (op_pooling.zig:16-35): no pads, no dilation, floor. */
int32_t zant_b200_pooling_output_shape(const size_t* x_shape, size_t x_rank,
                                       const size_t kernel[2], const size_t stride[2],
                                       size_t out_shape[4]);

/* get_onnx_maxpool_output_shape (op_pooling.zig:477-567). */
int32_t zant_b200_maxpool_output_shape(const size_t* x_shape, size_t x_rank,
                                       const size_t* kernel_shape, const size_t* strides,
                                       const size_t* dilations, const size_t* pads,
                                       int32_t auto_pad, int32_t ceil_mode,
                                       size_t out_shape[4]);

/* get_resize_output_shape (lib_shape_math.zig:78-104): exactly one of scales/sizes. */
int32_t zant_b200_resize_output_shape(const size_t* x_shape, size_t rank,
                                      const float* scales, size_t n_scales,
                                      const size_t* sizes, size_t n_sizes,
                                      size_t* out_shape);

/* Output shape of concatenate (lib_shape_math.zig:463-580): ranks are promoted with leading
 * ones to the largest rank; `out_shape` must hold that many entries; *out_rank receives it. */
int32_t zant_b200_concat_output_shape(const size_t* const* shapes, const size_t* ranks,
                                      size_t n_tensors, int64_t axis,
                                      size_t* out_shape, size_t* out_rank);

/* get_concatenate_output_shape (lib_shape_math.zig:582-629), the helper the generator calls:
 * all ranks must be equal (MismatchedRank) and non-axis dims must match (MismatchedShape). */
int32_t zant_b200_get_concatenate_output_shape(const size_t* const* shapes, const size_t* ranks,
                                               size_t n_tensors, int64_t axis, size_t* out_shape);

/* Contiguous sample shard of rank `rank` among `world` ranks: the first total%world ranks get
 * one extra sample. No reference counterpart (the reference is single-process). */
int32_t zant_b200_shard_range(size_t total, size_t world, size_t rank,
                              size_t* begin, size_t* count);

/* ------------------------------------------------------------------------------------------
 * FP32 operators (reference arithmetic: sequential fp32 accumulation, separate mul and add)
 * ---------------------------------------------------------------------------------------- */

/* tensMath.conv_lean = OnnxConvLean (op_convolution.zig:42-219, :228-331).
 * Y[n,m,oh,ow] = (sum over c,kh,kw in that order of Xpad*W) + B[m].  Pads are honoured only
 * when auto_pad is non-null ("NOTSET" reads pads[t,l,b,r]); a one-element stride/dilation is
 * used for both axes; group other than 1 returns InvalidDimensions; the output shape must
 * equal the computed one.  `bias`, `pads`, `dilations`, `auto_pad` may be NULL; group 0 = null. */
int32_t zant_b200_conv_f32(zant_ctx* ctx,
                           const float* x, const size_t* x_shape, size_t x_rank,
                           const float* w, const size_t* w_shape, size_t w_rank,
                           const float* bias, size_t bias_len,
                           float* y, const size_t* y_shape, size_t y_rank,
                           const size_t* stride, size_t n_stride,
                           const size_t* pads, size_t n_pads,
                           const size_t* dilations, size_t n_dil,
                           size_t group,
                           const char* auto_pad, size_t auto_pad_len);

/* tensMath.mat_mul_lean = lean_mat_mul (op_mat_mul.zig:92-172) with the checks of mat_mul
 * (:22-89).  Only the last two dimensions take part: Y[i,j] = sum_k A[i,k]*B[k,j], k ascending. */
int32_t zant_b200_mat_mul_f32(zant_ctx* ctx,
                              const float* a, const size_t* a_shape, size_t a_rank,
                              const float* b, const size_t* b_shape, size_t b_rank,
                              float* y, const size_t* y_shape, size_t y_rank);

/* tensMath.gemm_lean = lean_gemm (op_gemm.zig:91-185) with the checks of gemm (:15-87):
 * R = A'B'; R *= alpha; if C and beta != 0: R += C*beta, C broadcast over rows/cols of size 1.
 * Operands are 4-D [b,c,rows,cols]; as in the reference only the last two dims are multiplied. */
int32_t zant_b200_gemm_f32(zant_ctx* ctx,
                           const float* a, const size_t* a_shape, size_t a_rank,
                           const float* b, const size_t* b_shape, size_t b_rank,
                           const float* c, const size_t* c_shape, size_t c_rank,
                           float alpha, float beta, int32_t trans_a, int32_t trans_b,
                           float* y, const size_t* y_shape, size_t y_rank);

/* tensMath.gemm_lean as generated code calls it (src/codeGen/hardcoded/hardcoded_sentiment_it.zig:137):
 * lean_gemm (op_gemm.zig:91-185) without the rank check of the allocating wrapper.  Operands of rank 2..4
 * (C: 1..4) are taken as [1,..,1,rows,cols]; everything else as zant_b200_gemm_f32.  (The reference reads
 * shape[2] and shape[3] of rank-2 operands when C has to be broadcast, which is out of bounds; here that
 * case is the ONNX Gemm result.) */
int32_t zant_b200_gemm_lean_f32(zant_ctx* ctx,
                                const float* a, const size_t* a_shape, size_t a_rank,
                                const float* b, const size_t* b_shape, size_t b_rank,
                                const float* c, const size_t* c_shape, size_t c_rank,
                                float alpha, float beta, int32_t trans_a, int32_t trans_b,
                                float* y, const size_t* y_shape, size_t y_rank);

/* tensMath.onnx_maxpool_lean = lean_onnx_maxpool (op_pooling.zig:570-659).  SAME_* pads are
 * derived from the OUTPUT shape and the undilated kernel, as the reference does. */
int32_t zant_b200_maxpool_f32(zant_ctx* ctx,
                              const float* x, const size_t* x_shape, size_t x_rank,
                              float* y, const size_t* y_shape, size_t y_rank,
                              const size_t* kernel_shape, size_t n_kernel,
                              const size_t* strides, size_t n_strides,
                              const size_t* dilations, size_t n_dil,
                              const size_t* pads, size_t n_pads,
                              int32_t auto_pad);

/* tensMath.ReLU_lean = lean_ReLU (lib_activation_function_math.zig:22-28).  The reference
 * writes only positive inputs and relies on a zeroed output; this writes every element
 * (x > 0 ? x : 0), which is what the reference's callers observe. */
int32_t zant_b200_relu_f32(zant_ctx* ctx, const float* x, float* y, size_t n);

/* tensMath.leakyReLU_lean = lean_leakyReLU (lib_activation_function_math.zig:68-77). */
int32_t zant_b200_leaky_relu_f32(zant_ctx* ctx, const float* x, float slope, float* y, size_t n);

/* ONNX Clip on f32 (ReLU6 = clip(0,6)).  Not present in the reference. */
int32_t zant_b200_clip_f32(zant_ctx* ctx, const float* x, float lo, float hi, float* y, size_t n);

/* tensMath.transpose_onnx_lean (lib_shape_math.zig:1628-1753): y[out coords] = x[coords permuted];
 * `perm` NULL reverses the dimensions.  A perm of the wrong length, with an entry >= rank or with a
 * repeated entry is InvalidPermutation; an output of another rank InvalidRank.  Unlike the reference,
 * which overwrites the output's shape, the caller's y_shape must already be the permuted shape
 * (OutputTensorDifferentSize otherwise).  Any dtype (elements are moved, not interpreted). */
int32_t zant_b200_transpose_onnx(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                                 const size_t* perm, size_t n_perm, void* y, const size_t* y_shape, size_t y_rank);

/* tensMath.get_slice_output_shape / lean_slice_onnx (lib_shape_math.zig:1378-1495): ONNX Slice with
 * optional axes and steps (NULL = all axes in order / step 1).  starts/ends are clamped as the
 * reference does; starts.len != ends.len (here: one count `n` for all arrays) or an axis out of range is
 * InvalidSliceIndices, a zero step InvalidSliceStep.  `out_shape` receives x_rank entries. */
int32_t zant_b200_slice_output_shape(const size_t* x_shape, size_t x_rank, const int64_t* starts, const int64_t* ends, size_t n,
                                     const int64_t* axes, const int64_t* steps, size_t* out_shape);
/* The dimensions lean_slice_onnx itself writes into its output (lib_shape_math.zig:1445-1462).  They equal
 * get_slice_output_shape for positive steps; for a negative step the reference's two functions count
 * differently ((start - end) / |step| + 1 in the shape function, ceil((start - end - 1) / |step|) in the
 * operator), and zant_b200_slice_onnx follows the operator: its y_shape must be these dimensions. */
int32_t zant_b200_slice_lean_dims(const size_t* x_shape, size_t x_rank, const int64_t* starts, const int64_t* ends, size_t n,
                                  const int64_t* axes, const int64_t* steps, size_t* out_shape);
int32_t zant_b200_slice_onnx(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                             const int64_t* starts, const int64_t* ends, size_t n, const int64_t* axes, const int64_t* steps,
                             void* y, const size_t* y_shape, size_t y_rank);

/* tensMath.gather / lean_gather (lib_shape_math.zig:1217-1330): output shape = data.shape[:axis] ++
 * indices.shape ++ data.shape[axis+1:].  `indices` is a HOST array (the reference's Tensor(usize)).  Rank 0
 * data is InvalidRank, an axis outside [-rank, rank) InvalidAxis, an index >= the axis length
 * IndexOutOfBounds. */
int32_t zant_b200_gather(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                         const size_t* indices, const size_t* idx_shape, size_t idx_rank, int64_t axis,
                         void* y, const size_t* y_shape, size_t y_rank);

/* tensMath.get_unsqueeze_output_shape / unsqueeze_lean (lib_shape_math.zig:1933-2030): inserts
 * dimensions of size 1 at `axes` (positions in the OUTPUT; negative values count from its end).  An axis
 * outside the output rank is AxisOutOfBounds, a repeated one DuplicateAxis.  `out_shape` receives
 * x_rank + n_axes entries.  The data is copied unchanged. */
int32_t zant_b200_unsqueeze_output_shape(const size_t* x_shape, size_t x_rank, const int64_t* axes, size_t n_axes, size_t* out_shape);
int32_t zant_b200_unsqueeze(zant_ctx* ctx, int32_t dtype, const void* x, const size_t* x_shape, size_t x_rank,
                            const int64_t* axes, size_t n_axes, void* y, const size_t* y_shape, size_t y_rank);

/* tensMath.shape_onnx / lean_shape_onnx / get_shape_output_shape (lib_shape_math.zig:1836-1931): the
 * dimensions [start, end) of a shape as int64 values, written to the HOST array `out` (x_rank entries of
 * room); no device work.  has_start / has_end = 0 stand for the absent ONNX attributes. */
int32_t zant_b200_shape_onnx(const size_t* x_shape, size_t x_rank, int32_t has_start, int64_t start, int32_t has_end, int64_t end,
                             int64_t* out, size_t* out_len);

/* tensMath.sigmoid_lean (lib_activation_function_math.zig:107-122): 1 / (1 + exp(-x)). */
int32_t zant_b200_sigmoid_f32(zant_ctx* ctx, const float* x, float* y, size_t n);
/* tensMath.softmax_lean = lean_softmax (lib_activation_function_math.zig:154-187): x is [rows][cols];
 * per row: maximum, exp(x - max) summed in index order, division by the sum. */
int32_t zant_b200_softmax_f32(zant_ctx* ctx, const float* x, float* y, size_t rows, size_t cols);
/* tensMath.tanh_lean / ceil_lean (lib_elementWise_math.zig:452-456, 471-480; ceil passes NaN and
 * infinities through). */
int32_t zant_b200_tanh_f32(zant_ctx* ctx, const float* x, float* y, size_t n);
int32_t zant_b200_ceil_f32(zant_ctx* ctx, const float* x, float* y, size_t n);
/* tensMath.mul_lean / div_lean (lib_elementWise_math.zig:392-427): element-wise on tensors of equal
 * size; different sizes return MismatchedShape as TensMath.mul / div do. */
int32_t zant_b200_mul_f32(zant_ctx* ctx, const float* a, size_t n_a, const float* b, size_t n_b, float* y);
int32_t zant_b200_div_f32(zant_ctx* ctx, const float* a, size_t n_a, const float* b, size_t n_b, float* y);

/* tensMath.sum_tensors_lean = lean_sum_tensors (lib_elementWise_math.zig:70-210): equal
 * sizes add element-wise; otherwise NumPy right-aligned broadcasting up to rank 4. */
int32_t zant_b200_sum_tensors_f32(zant_ctx* ctx,
                                  const float* a, const size_t* a_shape, size_t a_rank,
                                  const float* b, const size_t* b_shape, size_t b_rank,
                                  float* y, const size_t* y_shape, size_t y_rank);

/* tensMath.sum_tensor_list_lean = lean_sum_tensor_list (lib_elementWise_math.zig:243-257):
 * y = t0; y += t1; ... in list order.  All tensors hold `n` elements. */
int32_t zant_b200_sum_tensor_list_f32(zant_ctx* ctx, const float* const* tensors,
                                      size_t n_tensors, float* y, size_t n);

/* tensMath.concatenate (lib_shape_math.zig:307-445, :463-580).  The output buffer is the
 * caller's (shape from zant_b200_concat_output_shape). */
int32_t zant_b200_concatenate(zant_ctx* ctx, int32_t dtype,
                              const void* const* tensors, const size_t* const* shapes,
                              const size_t* ranks, size_t n_tensors, int64_t axis,
                              void* y, const size_t* y_shape, size_t y_rank);

/* tensMath.resize with mode "nearest" (lib_shape_math.zig:22-76, :106-161): coordinate modes
 * "half_pixel", "align_corners", anything else = asymmetric; index = round-half-away then
 * clamp.  Other modes return UnsupportedMode ("linear"/"cubic": ZANT_E_UNSUPPORTED). */
int32_t zant_b200_resize(zant_ctx* ctx, int32_t dtype,
                         const void* x, const size_t* x_shape, size_t rank,
                         const char* mode, size_t mode_len,
                         const float* scales, size_t n_scales,
                         const size_t* sizes, size_t n_sizes,
                         const char* coord_mode, size_t coord_mode_len,
                         void* y, const size_t* y_shape, size_t y_rank);

/* tensMath.reduce_mean_lean = lean_reduce_mean (lib_reduction_math.zig:87-268): sequential
 * fp32 sum in the reference's visiting order, then one division by the count. */
int32_t zant_b200_reduce_mean_f32(zant_ctx* ctx,
                                  const float* x, const size_t* x_shape, size_t x_rank,
                                  float* y, const size_t* y_shape, size_t y_rank,
                                  const int64_t* axes, size_t n_axes,
                                  int32_t keepdims, int32_t noop_with_empty_axes);

/* tensMath.reshape_lean (lib_shape_math.zig:1139-1209): resolves 0 (copy input dim) and
 * SIZE_MAX (the generator's encoding of -1), writes the resolved shape to `y_shape_out`
 * (new_rank entries) and copies the data unchanged. */
int32_t zant_b200_reshape(zant_ctx* ctx, int32_t dtype,
                          const void* x, const size_t* x_shape, size_t x_rank,
                          const size_t* new_shape, size_t new_rank,
                          void* y, size_t* y_shape_out);

/* ------------------------------------------------------------------------------------------
 * Quantized operators (no counterpart in the reference tree; ONNX definitions).
 * All float math is IEEE fp32, round-to-nearest-even, no fused multiply-add.
 *   rne(v)   = nearest integer, ties to even, of v clamped to [-512, 511]
 *   sat(t)   = clamp to the output type's range
 * ---------------------------------------------------------------------------------------- */

/* ONNX QuantizeLinear, per tensor: y = sat(rne(x / scale) + zp).  out_dtype I8 or U8. */
int32_t zant_b200_quantize_linear(zant_ctx* ctx, const float* x, size_t n,
                                  float scale, int32_t zero_point,
                                  int32_t out_dtype, void* y);

/* ONNX DequantizeLinear, per tensor: y = float(q - zp) * scale.  in_dtype I8, U8 or I32. */
int32_t zant_b200_dequantize_linear(zant_ctx* ctx, int32_t in_dtype, const void* q, size_t n,
                                    float scale, int32_t zero_point, float* y);

/* ONNX QLinearConv (NCHW, groups allowed, depthwise = group == C):
 *   acc = sum (x - x_zp) * (w - w_zp[m]) + bias[m]            exact int32
 *   M[m] = (x_scale * w_scale[m]) / y_scale                    one multiply, one divide
 *   y   = sat(rne(float(acc) * M[m]) + y_zp), then the fused activation.
 * Padding contributes (x_zp - x_zp) = 0.  w is int8 [M, C/group, KH, KW]; w_scale / w_zp hold
 * n_w_scale entries (1 = per tensor, M = per output channel); bias may be NULL.
 * Pads follow ONNX: explicit pads[t,l,b,r] unless auto_pad is SAME_UPPER/SAME_LOWER/VALID. */
int32_t zant_b200_qlinearconv(zant_ctx* ctx,
                              int32_t x_dtype, const void* x, const size_t* x_shape, size_t x_rank,
                              float x_scale, int32_t x_zp,
                              const int8_t* w, const size_t* w_shape, size_t w_rank,
                              const float* w_scale, const int32_t* w_zp, size_t n_w_scale,
                              float y_scale, int32_t y_zp,
                              const int32_t* bias, size_t bias_len,
                              int32_t y_dtype, void* y, const size_t* y_shape, size_t y_rank,
                              const size_t* stride, size_t n_stride,
                              const size_t* pads, size_t n_pads,
                              const size_t* dilations, size_t n_dil,
                              size_t group, int32_t auto_pad, int32_t activation);

/* ONNX QLinearMatMul on 2-D operands: A [M,K] (I8/U8), B int8 [K,N], per-tensor or per-column
 * b_scale / b_zp (n_b_scale = 1 or N); optional int32 bias[N] (an extension used for fused
 * fully-connected layers; NULL for plain ONNX).  Same requantisation as QLinearConv. */
int32_t zant_b200_qlinearmatmul(zant_ctx* ctx,
                                int32_t a_dtype, const void* a, const size_t* a_shape, size_t a_rank,
                                float a_scale, int32_t a_zp,
                                const int8_t* b, const size_t* b_shape, size_t b_rank,
                                const float* b_scale, const int32_t* b_zp, size_t n_b_scale,
                                float y_scale, int32_t y_zp,
                                const int32_t* bias, size_t bias_len,
                                int32_t y_dtype, void* y, const size_t* y_shape, size_t y_rank,
                                int32_t activation);

/* QLinearConv on channels-last tensors: x is [N, H, W, C], y is [N, OH, OW, M]; w stays the ONNX
 * [M, C, KH, KW].  The reference has no channels-last operator (its tensors are NCHW,
 * src/Core/Tensor/TensorMath/op_convolution.zig:42); this entry point serves callers that keep
 * activations channels-last between layers, the layout in which a TMA box of the input is a tensor-core
 * operand as it lands.  Arithmetic, remaining arguments and error codes are those of
 * zant_b200_qlinearconv.  Shapes the channels-last kernel does not take (group != 1, stride != 1,
 * C % 64 != 0, M % 16 != 0, non-zero weight zero points, padding together with x_zp != 0) return
 * ZANT_E_UNSUPPORTED: there is no second code path behind this entry point. */
int32_t zant_b200_qlinearconv_nhwc(zant_ctx* ctx,
                                   int32_t x_dtype, const void* x, const size_t* x_shape, size_t x_rank,
                                   float x_scale, int32_t x_zp,
                                   const int8_t* w, const size_t* w_shape, size_t w_rank,
                                   const float* w_scale, const int32_t* w_zp, size_t n_w_scale,
                                   float y_scale, int32_t y_zp,
                                   const int32_t* bias, size_t bias_len,
                                   int32_t y_dtype, void* y, const size_t* y_shape, size_t y_rank,
                                   const size_t* stride, size_t n_stride,
                                   const size_t* pads, size_t n_pads,
                                   const size_t* dilations, size_t n_dil,
                                   size_t group, int32_t auto_pad, int32_t activation);

/* QLinearConv for callers that cannot allocate device memory (no counterpart in the reference:
 * its operators run on the CPU heap).  Think of an inference loop whose memory was handed out
 * once at start-up, a latency-critical thread that must avoid cudaMalloc's device-wide
 * synchronisation, or a port of Z-Ant's generated code, which owns only static arrays.  The
 * regular entry point needs a context, and a context owns a cudaMalloc'd arena; this one takes
 * a cudaStream_t (as void*, NULL = default stream) instead and allocates nothing.  The
 * per-channel requantisation constants that the kernel reads besides x, w, bias and y are kept
 * in a fixed device array inside the library (32 KiB per GPU, held until the process exits).
 *   - same arithmetic, argument meaning and error codes as zant_b200_qlinearconv;
 *   - x, w, bias, y: DEVICE pointers of the current device (another GPU's memory is refused with
 *     ZANT_E_INVALID_INPUT); w_scale, w_zp: host arrays;
 *   - at most 4096 output channels, otherwise ZANT_E_TOO_LARGE;
 *   - the first call on a device resolves the array's device address;
 *   - never call it on a stream that is being captured (ZANT_E_UNSUPPORTED): every call copies its
 *     per-channel constants from host buffers of the calling thread into the array;
 *   - all calls on a device share the array, so calls whose kernels could overlap on the GPU
 *     race: keep them on one stream or order them with events;
 *   - it returns once the small constant copy (from pageable host memory, so it may wait for
 *     earlier work of the stream) is handed over and the kernel is enqueued; it does not wait
 *     for the kernel. */
int32_t zant_b200_qlinearconv_noalloc(void* cuda_stream,
                                      int32_t x_dtype, const void* x, const size_t* x_shape, size_t x_rank,
                                      float x_scale, int32_t x_zp,
                                      const int8_t* w, const size_t* w_shape, size_t w_rank,
                                      const float* w_scale, const int32_t* w_zp, size_t n_w_scale,
                                      float y_scale, int32_t y_zp,
                                      const int32_t* bias, size_t bias_len,
                                      int32_t y_dtype, void* y, const size_t* y_shape, size_t y_rank,
                                      const size_t* stride, size_t n_stride,
                                      const size_t* pads, size_t n_pads,
                                      const size_t* dilations, size_t n_dil,
                                      size_t group, int32_t auto_pad, int32_t activation);

/* Quantized Add (QLinearAdd / QDQ residual), equal shapes:
 *   y = sat(rne((float(a - a_zp) * a_s + float(b - b_zp) * b_s) / y_s) + y_zp). */
int32_t zant_b200_qlinearadd(zant_ctx* ctx, int32_t dtype,
                             const void* a, float a_scale, int32_t a_zp,
                             const void* b, float b_scale, int32_t b_zp,
                             float y_scale, int32_t y_zp, void* y, size_t n, int32_t activation);

/* Quantized GlobalAveragePool over H,W of NCHW:
 *   sum exact int32 of (q - x_zp); y = sat(rne((float(sum) * x_s) / float(H*W) / y_s) + y_zp). */
int32_t zant_b200_qlinear_global_avgpool(zant_ctx* ctx, int32_t dtype,
                                         const void* x, const size_t* x_shape, size_t x_rank,
                                         float x_scale, int32_t x_zp,
                                         float y_scale, int32_t y_zp, void* y);

/* MaxPool on raw int8/uint8 codes (monotone, so scale and zero point carry over).  Same
 * window rules as zant_b200_maxpool_f32; a window with no valid tap yields the type minimum. */
int32_t zant_b200_maxpool_q8(zant_ctx* ctx, int32_t dtype,
                             const void* x, const size_t* x_shape, size_t x_rank,
                             void* y, const size_t* y_shape, size_t y_rank,
                             const size_t* kernel_shape, size_t n_kernel,
                             const size_t* strides, size_t n_strides,
                             const size_t* dilations, size_t n_dil,
                             const size_t* pads, size_t n_pads,
                             int32_t auto_pad);

/* Element-wise requantisation through a 256-entry table indexed by the raw code
 * (unsigned view of the byte): y[i] = lut[(uint8_t)x[i]].  Used for LeakyReLU / ReLU /
 * rescale between QDQ tensors, where the table is built on the host from the pinned formula. */
int32_t zant_b200_lut_q8(zant_ctx* ctx, const void* x, const uint8_t lut[256], void* y, size_t n);

/* ------------------------------------------------------------------------------------------
 * Plan: the run-time form of a generated predict() (src/codeGen/predict.zig:23-70).  One
 * device buffer per graph tensor at a fixed offset of one cudaMalloc'd arena (the analogue
 * of the generator's one static array per tensor, predict.zig:110-142, :265-272), constants
 * uploaded once, nodes run in insertion order (the generator emits them in ready-set order).
 * ---------------------------------------------------------------------------------------- */

typedef enum zant_op {
    ZANT_OP_CONV = 1,
    ZANT_OP_MATMUL = 2,
    ZANT_OP_GEMM = 3,
    ZANT_OP_MAXPOOL = 4,
    ZANT_OP_RELU = 5,
    ZANT_OP_LEAKY_RELU = 6,
    ZANT_OP_ADD = 7,
    ZANT_OP_CONCAT = 8,
    ZANT_OP_RESIZE = 9,
    ZANT_OP_REDUCE_MEAN = 10,
    ZANT_OP_RESHAPE = 11,
    ZANT_OP_CLIP = 12,
    ZANT_OP_SIGMOID = 13,
    ZANT_OP_SOFTMAX = 14,           /* 2-D input, rows normalised */
    ZANT_OP_TANH = 15,
    ZANT_OP_CEIL = 16,
    ZANT_OP_MUL = 17,               /* equal sizes */
    ZANT_OP_DIV = 18,
    ZANT_OP_TRANSPOSE = 19,         /* attrs.perm */
    ZANT_OP_SLICE = 27,             /* attrs.slice_* */
    ZANT_OP_GATHER = 28,            /* inputs: data, indices (I32 initializer); attrs.axis */
    ZANT_OP_QUANTIZE_LINEAR = 20,
    ZANT_OP_DEQUANTIZE_LINEAR = 21,
    ZANT_OP_QLINEAR_CONV = 22,
    ZANT_OP_QLINEAR_MATMUL = 23,
    ZANT_OP_QLINEAR_ADD = 24,
    ZANT_OP_QLINEAR_GLOBAL_AVGPOOL = 25,
    ZANT_OP_LUT_Q8 = 26
} zant_op;

/* Attributes of one node; unused fields are ignored.  n_* = 0 means "null" where the
 * reference takes an optional slice. */
typedef struct zant_node_attrs {
    size_t kernel_shape[2];
    size_t strides[2];   size_t n_strides;
    size_t dilations[2]; size_t n_dilations;
    size_t pads[4];      size_t n_pads;
    size_t group;        /* 0 = null */
    int32_t auto_pad;    /* zant_auto_pad; for Conv: -1 = null (pads ignored, as the reference) */
    float alpha, beta;   /* Gemm; LeakyRelu slope in alpha; Clip lo/hi in alpha/beta */
    int32_t trans_a, trans_b;
    int64_t axis;        /* Concat */
    int64_t axes[4];     size_t n_axes;  /* ReduceMean */
    int32_t keepdims, noop_with_empty_axes;
    float scales[4];     size_t n_scales; /* Resize */
    int32_t coord_mode;  /* Resize: 0 half_pixel, 1 align_corners, 2 asymmetric */
    /* quantisation parameters */
    float x_scale;  int32_t x_zp;
    float b_scale;  int32_t b_zp;   /* second operand of QLinearAdd */
    float y_scale;  int32_t y_zp;
    int32_t activation;             /* zant_qact */
    /* Transpose */
    int64_t perm[8];     size_t n_perm;          /* n_perm = 0: reverse the dimensions */
    /* Slice: n_slice entries; has_* = 0 means the optional ONNX input is absent */
    int64_t slice_starts[8], slice_ends[8], slice_axes[8], slice_steps[8];
    size_t n_slice; int32_t slice_has_axes, slice_has_steps;
    /* QLinearConv: 1 = x is [N,H,W,C] and y is [N,OH,OW,M] (w stays [M,C,KH,KW]); shapes the
     * channels-last kernel does not take make zant_b200_plan_finalize return ZANT_E_UNSUPPORTED */
    int32_t channels_last;
} zant_node_attrs;

int32_t zant_b200_plan_create(zant_ctx* ctx, zant_plan** out);
int32_t zant_b200_plan_destroy(zant_plan* plan);

/* Declares a graph tensor.  `const_data` non-NULL marks an initializer (host pointer, copied
 * at this call; the analogue of static_parameters.zig).  Returns the tensor id in *id. */
int32_t zant_b200_plan_tensor(zant_plan* plan, int32_t dtype, const size_t* shape, size_t rank,
                              const void* const_data, int32_t* id);

/* Appends a node.  Input order follows the ONNX operator (QLinearConv: x, w, w_scale, w_zp,
 * bias with per-tensor x/y parameters in attrs; w_scale is an F32 tensor, w_zp an I32 tensor;
 * -1 for an absent optional input). */
int32_t zant_b200_plan_node(zant_plan* plan, int32_t op,
                            const int32_t* inputs, size_t n_inputs,
                            const int32_t* outputs, size_t n_outputs,
                            const zant_node_attrs* attrs);

/* Marks the graph input and output, validates every node's shapes with the same rules as
 * the single-op entry points, assigns arena offsets, uploads constants, prepares weights and
 * selects fused kernels.  `fuse` = 0 keeps one kernel per node (the reference's structure). */
int32_t zant_b200_plan_finalize(zant_plan* plan, int32_t input_id, int32_t output_id, int32_t fuse);

/* Runs the plan once: the analogue of predict(input, shape, len, &result)
 * (src/codeGen/predict.zig:34-40).  `input`/`output` may be host or device pointers.
 * Pageable host buffers: the call returns when the result is in `output`.  Device buffers, or
 * page-locked (pinned) host buffers on both sides: the call only enqueues work on the context's
 * stream; zant_b200_ctx_synchronize waits for it and reports device-side errors. */
int32_t zant_b200_plan_run(zant_plan* plan, const void* input, void* output);

/* Captures the plan's launches into a CUDA graph (enable != 0) or drops it (enable == 0).  With a
 * graph, zant_b200_plan_run replays all steps with one cudaGraphLaunch: what the reference's
 * generated predict() does with a fixed sequence of calls, minus the per-launch cost, which is
 * what batch-1 latency consists of.  Inputs and outputs always pass through the arena's own input and
 * output buffers then (device buffers are copied in and out).  Results are identical to the
 * un-captured run; per-step profiling falls back to separate launches while it is enabled. */
int32_t zant_b200_plan_use_graph(zant_plan* plan, int32_t enable);

/* Bytes of the plan's arena and number of kernels one run launches. */
size_t zant_b200_plan_arena_bytes(zant_plan* plan);
int32_t zant_b200_plan_launches_per_run(zant_plan* plan);
/* Number of launch steps of a finalized plan and the name of step i ("QLinearConv", ...). */
int32_t zant_b200_plan_step_count(zant_plan* plan);
const char* zant_b200_plan_step_name(zant_plan* plan, int32_t step);
/* Algorithmic work of step i: multiply-accumulates of the contractions it covers, and bytes = every tensor
 * that crosses the step's boundary (inputs and initializers read, results written), each counted once at its
 * storage type; tensors interior to a fused step do not count.  These are the numerators of the roofline
 * figures the benchmark reports per step.  Either pointer may be NULL. */
int32_t zant_b200_plan_step_cost(zant_plan* plan, int32_t step, double* macs, double* bytes);
/* Per-step device timing: when enabled, every run records one CUDA event before each step and
 * one after the last on the context's stream (no synchronisation is added).  _read drains the
 * stream, adds the elapsed milliseconds of every recorded run to sum_ms[step] (step_count
 * entries, zeroed by the caller), stores the number of runs in *runs and clears the record. */
int32_t zant_b200_plan_profile(zant_plan* plan, int32_t enable);
int32_t zant_b200_plan_profile_read(zant_plan* plan, float* sum_ms, int32_t* runs);
/* Device pointer of a tensor's arena buffer (for tests that inspect intermediates). */
void* zant_b200_plan_tensor_ptr(zant_plan* plan, int32_t id);
/* Copies a tensor's current contents to `host_dst` (tensor-sized) after draining the stream. */
int32_t zant_b200_plan_read_tensor(zant_plan* plan, int32_t id, void* host_dst);

/* ------------------------------------------------------------------------------------------
 * Sample-sharded predict over several GPUs of one machine.  The reference bakes the batch into the
 * generated predict() (src/codeGen/predict.zig:34-40, :317-336) and is single-threaded; this is the
 * extension that splits one host batch across devices.  Samples are independent, so there is no
 * collective: device i gets the contiguous samples of zant_b200_shard_range(n, world, i) and writes
 * its results into the matching slice of the caller's output buffer.  One context, one stream, one
 * arena and one host worker thread per device.
 * ---------------------------------------------------------------------------------------- */
typedef struct zant_multi zant_multi;

/* `devices` NULL or n_devices 0: the comma-separated list in the environment variable
 * ZANT_B200_DEVICES ("0,2,3"), else every visible device.  A device may appear more than once (two
 * contexts on one GPU).  `arena_bytes` as for zant_b200_ctx_create. */
int32_t zant_b200_multi_create(const int32_t* devices, size_t n_devices, size_t arena_bytes, zant_multi** out);
/* Destroys the contexts and stops the workers; destroy the shards' plans first. */
int32_t zant_b200_multi_destroy(zant_multi* multi);
size_t zant_b200_multi_size(zant_multi* multi);
/* Context of shard i: build that shard's plan on it. */
zant_ctx* zant_b200_multi_ctx(zant_multi* multi, size_t i);
/* Registers the finalized plan of shard i.  Its batch (leading dimension of its input and output)
 * must be the number of samples zant_b200_shard_range gives shard i for the batches later passed
 * to zant_b200_predict_sharded. */
int32_t zant_b200_multi_set_plan(zant_multi* multi, size_t i, zant_plan* plan);
/* predict() for `n_samples` samples in HOST buffers (pageable or pinned): all shards run at once,
 * the call returns when every result is in `host_out`.  `status_per_device` (zant_b200_multi_size
 * entries, may be NULL) receives each shard's status; the return value is the first failure, so one
 * failing device is reported without hiding what the others did. */
int32_t zant_b200_predict_sharded(zant_multi* multi, const void* host_in, void* host_out, size_t n_samples,
                                  int32_t* status_per_device);

#ifdef __cplusplus
}
#endif
#endif /* ZANT_B200_H */
