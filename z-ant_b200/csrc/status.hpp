// Status names, per-thread last-error text and the log hook shared by every entry point.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/zant_b200.h"

namespace zb {

inline const char* status_name(int32_t s) {
    switch (s) {
        case ZANT_OK: return "OK";
        case ZANT_E_INVALID_DIMENSIONS: return "InvalidDimensions";
        case ZANT_E_MEM_ERROR: return "MemError";
        case ZANT_E_INPUT_TENSOR_DIFFERENT_SIZE: return "InputTensorDifferentSize";
        case ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE: return "InputTensorDifferentShape";
        case ZANT_E_INPUT_TENSORS_WRONG_SHAPE: return "InputTensorsWrongShape";
        case ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE: return "OutputTensorDifferentSize";
        case ZANT_E_TOO_SMALL_OUTPUT_TYPE: return "TooSmallOutputType";
        case ZANT_E_INPUT_TENSOR_DIMENSION_MISMATCH: return "InputTensorDimensionMismatch";
        case ZANT_E_WRONG_STRIDE: return "WrongStride";
        case ZANT_E_INCOMPATIBLE_BROADCAST_SHAPES: return "IncompatibleBroadcastShapes";
        case ZANT_E_EMPTY_TENSOR_LIST: return "EmptyTensorList";
        case ZANT_E_DIVISION_ERROR: return "DivisionError";
        case ZANT_E_INVALID_PADDING: return "InvalidPadding";
        case ZANT_E_INVALID_AXES: return "InvalidAxes";
        case ZANT_E_TENSOR_NOT_INITIALIZED: return "TensorNotInitialized";
        case ZANT_E_INPUT_ARRAY_WRONG_TYPE: return "InputArrayWrongType";
        case ZANT_E_INPUT_ARRAY_WRONG_SIZE: return "InputArrayWrongSize";
        case ZANT_E_EMPTY_TENSOR: return "EmptyTensor";
        case ZANT_E_ZERO_SIZE_TENSOR: return "ZeroSizeTensor";
        case ZANT_E_INVALID_SLICE_INDICES: return "InvalidSliceIndices";
        case ZANT_E_INVALID_SLICE_STEP: return "InvalidSliceStep";
        case ZANT_E_INVALID_AXIS: return "InvalidAxis";
        case ZANT_E_DUPLICATE_AXIS: return "DuplicateAxis";
        case ZANT_E_INVALID_RANK: return "InvalidRank";
        case ZANT_E_INVALID_PERMUTATION: return "InvalidPermutation";
        case ZANT_E_AXIS_OUT_OF_BOUNDS: return "AxisOutOfBounds";
        case ZANT_E_MISMATCHED_RANK: return "MismatchedRank";
        case ZANT_E_MISMATCHED_SHAPE: return "MismatchedShape";
        case ZANT_E_INDEX_OUT_OF_BOUNDS: return "IndexOutOfBounds";
        case ZANT_E_INVALID_INPUT: return "InvalidInput";
        case ZANT_E_UNSUPPORTED_MODE: return "UnsupportedMode";
        case ZANT_E_UNSUPPORTED_DIMENSION: return "UnsupportedDimension";
        case ZANT_E_CUDA: return "Cuda";
        case ZANT_E_CUDA_UNAVAILABLE: return "CudaUnavailable";
        case ZANT_E_NULL_POINTER: return "NullPointer";
        case ZANT_E_UNSUPPORTED: return "Unsupported";
        case ZANT_E_ARENA_EXHAUSTED: return "ArenaExhausted";
        case ZANT_E_BAD_HANDLE: return "BadHandle";
        case ZANT_E_DEVICE_TIMEOUT: return "DeviceTimeout";
        case ZANT_E_TOO_LARGE: return "TooLarge";
        default: return "UnknownStatus";
    }
}

inline std::string& last_error_ref() {
    static thread_local std::string e;
    return e;
}

using log_fn_t = void (*)(char*);
inline log_fn_t& log_fn_ref() {
    static log_fn_t fn = nullptr;
    return fn;
}

// Environment switch: set and neither empty nor "0".
inline bool env_flag(const char* name) {
    const char* v = std::getenv(name);
    return v && *v && std::strcmp(v, "0") != 0;
}

// One line per event to the installed callback; without a callback, to stderr when the environment
// variable ZANT_B200_LOG is set (the run-time analogue of the generator's -Dlog option,
// src/codeGen/math_handler.zig:35-43).
inline void log_line(const char* fmt, ...) {
    log_fn_t fn = log_fn_ref();
    static const bool to_stderr = env_flag("ZANT_B200_LOG");
    if (!fn && !to_stderr) return;
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (fn) fn(buf);
    else std::fprintf(stderr, "%s\n", buf);
}

// Records a failure (status + message) for zant_b200_last_error() and returns the status.
inline int32_t fail(int32_t st, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = std::string(status_name(st)) + ": " + buf;
    log_line("zant_b200 error %s", last_error_ref().c_str());
    return st;
}

}  // namespace zb
