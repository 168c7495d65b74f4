// zant_b200_qlinearconv_noalloc: QLinearConv for callers that must not allocate device memory.
//
// Some users of this library run where cudaMalloc is off the table: an inference loop with a
// fixed memory budget that was carved up at start-up, a real-time thread that cannot afford
// cudaMalloc's implicit device synchronisation, or a deployment modelled on Z-Ant's own
// generated code, which owns nothing but static arrays.  The regular entry point
// (zant_b200_qlinearconv) needs a context, and creating a context allocates an arena.  This
// variant needs no context and allocates nothing: the per-channel requantisation constants that
// the kernel reads besides its inputs and outputs live in the fixed device array below.
//
// Limits and rules for the caller
//   * at most ZANT_NOALLOC_MAX_CHANNELS output channels; more is rejected with ZANT_E_TOO_LARGE;
//   * x, w, bias and y must be DEVICE pointers of the current device (nothing is staged; memory
//     of another GPU is refused with ZANT_E_INVALID_INPUT); w_scale / w_zp are small HOST arrays;
//   * the first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress);
//   * no call may be made on a stream that is being captured: every call copies its constants
//     from host buffers of the calling thread into the array, and a captured copy would re-read
//     those buffers at every replay.  Such a call is refused with ZANT_E_UNSUPPORTED;
//   * the call returns once the constants have been handed to the driver (a small copy from
//     pageable host memory, which may wait for earlier work of the stream) and the kernel is
//     enqueued; it does not wait for the kernel;
//   * every call on a device shares the one array and overwrites the constants it needs, so two
//     calls whose kernels may overlap on the GPU (different streams, no dependency) race on it:
//     serialise them, e.g. by issuing them on one stream;
//   * the array holds 8 * ZANT_NOALLOC_MAX_CHANNELS bytes of every GPU that loads this library
//     until the process exits.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/zant_b200.h"
#include "geometry.hpp"
#include "kernels_q8.cuh"
#include "status.hpp"

#define ZANT_NOALLOC_MAX_CHANNELS 4096

namespace {

// [0, MAX) float multipliers M[m] = (x_scale * w_scale[m]) / y_scale, then [MAX, 2*MAX) int32
// weight zero points.  In host code this name is only a handle for cudaGetSymbolAddress; it is
// not an address the device can use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[8 * ZANT_NOALLOC_MAX_CHANNELS];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device, resolved once per device.
int32_t scratch_address(int device, void** out) {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (device < 0 || device >= kMaxDevices) return zb::fail(ZANT_E_INVALID_INPUT, "device index %d", device);
    if (!g_scratch_addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return zb::fail(ZANT_E_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return ZANT_OK;
}

// Device memory of `device` (or managed memory, which every device may touch).
bool device_pointer(const void* p, int device) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeManaged || (a.type == cudaMemoryTypeDevice && a.device == device);
}

}  // namespace

extern "C" int32_t zant_b200_qlinearconv_noalloc(
    void* cuda_stream, int32_t x_dtype, const void* x, const size_t* x_shape, size_t x_rank, float x_scale, int32_t x_zp,
    const int8_t* w, const size_t* w_shape, size_t w_rank, const float* w_scale, const int32_t* w_zp, size_t n_w_scale,
    float y_scale, int32_t y_zp, const int32_t* bias, size_t bias_len, int32_t y_dtype, void* y, const size_t* y_shape,
    size_t y_rank, const size_t* stride, size_t n_stride, const size_t* pads, size_t n_pads, const size_t* dilations,
    size_t n_dil, size_t group, int32_t auto_pad, int32_t activation) {
    using namespace zb;
    if (!x || !w || !y || !x_shape || !w_shape || !y_shape || !w_scale) return fail(ZANT_E_NULL_POINTER, "x, w, y, shapes and w_scale are required");
    const bool q8x = x_dtype == ZANT_I8 || x_dtype == ZANT_U8, q8y = y_dtype == ZANT_I8 || y_dtype == ZANT_U8;
    if (!q8x || !q8y) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearConv tensors must be int8 or uint8");
    if (int32_t zs = check_zero_point(x_dtype, x_zp, "QLinearConv x")) return zs;
    ConvGeom g;
    int32_t st = conv_resolve_onnx(x_shape, x_rank, w_shape, w_rank, y_shape, y_rank, stride, n_stride, pads, n_pads, dilations, n_dil, group, auto_pad, g);
    if (st != ZANT_OK) return st;
    if (g.M > ZANT_NOALLOC_MAX_CHANNELS)
        return fail(ZANT_E_TOO_LARGE, "%d output channels exceed the no-allocation limit of %d; use zant_b200_qlinearconv", g.M, ZANT_NOALLOC_MAX_CHANNELS);
    if (n_w_scale != 1 && n_w_scale != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "w_scale holds %zu values for %d filters", n_w_scale, g.M);
    if (bias && bias_len != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "bias holds %zu values for %d filters", bias_len, g.M);
    if (activation < ZANT_QACT_NONE || activation > ZANT_QACT_RELU6) return fail(ZANT_E_INVALID_INPUT, "activation %d", activation);

    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(ZANT_E_CUDA_UNAVAILABLE, "no CUDA device (%s); there is no CPU fallback", cudaGetErrorString(e)); }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(stream, &capture);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(ZANT_E_CUDA, "cudaStreamIsCapturing: %s", cudaGetErrorString(e)); }
    if (capture != cudaStreamCaptureStatusNone)
        return fail(ZANT_E_UNSUPPORTED, "the stream is being captured: this entry point copies per-call constants from host buffers and cannot be recorded");
    if (!device_pointer(x, device) || !device_pointer(w, device) || !device_pointer(y, device) || (bias && !device_pointer(bias, device)))
        return fail(ZANT_E_INVALID_INPUT, "x, w, bias and y must be device pointers of the current device %d: this entry point stages nothing", device);
    void* scratch = nullptr;
    st = scratch_address(device, &scratch);
    if (st != ZANT_OK) return st;

    // Host-side constants in fixed thread-local buffers (no heap, no device allocation), then into the shared array.
    // Nothing in the array has to start at zero: every slot the kernel reads is rewritten here.
    static thread_local float h_mult[ZANT_NOALLOC_MAX_CHANNELS];
    static thread_local int32_t h_wzp[ZANT_NOALLOC_MAX_CHANNELS];
    for (int m = 0; m < g.M; ++m) {
        volatile float xw = x_scale * w_scale[n_w_scale == 1 ? 0 : m];
        h_mult[m] = xw / y_scale;
        h_wzp[m] = w_zp ? w_zp[n_w_scale == 1 ? 0 : m] : 0;
    }
    float* d_mult = reinterpret_cast<float*>(scratch);
    int32_t* d_wzp = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(scratch) + 4 * ZANT_NOALLOC_MAX_CHANNELS);
    e = cudaMemcpyAsync(d_mult, h_mult, sizeof(float) * g.M, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_wzp, h_wzp, sizeof(int32_t) * g.M, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail(ZANT_E_CUDA, "copy of requantisation constants: %s", cudaGetErrorString(e));

    QConvArgs p{};
    p.x = x; p.w = w; p.y = y; p.mult = d_mult; p.w_zp = d_wzp; p.bias = bias;
    p.x_zp = x_zp; p.rq = Requant{y_scale, y_zp, activation}; p.g = g;
    const size_t total = (size_t)g.N * g.M * g.OH * g.OW;
    if (total == 0) return ZANT_OK;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
    size_t blocks = (total + 127) / 128;
    if (blocks > (size_t)sms * 32) blocks = (size_t)sms * 32;
    const bool xu = x_dtype == ZANT_U8, yu = y_dtype == ZANT_U8;
    if (xu && yu) qconv_nchw_generic<true, true><<<(unsigned)blocks, 128, 0, stream>>>(p);
    else if (xu) qconv_nchw_generic<true, false><<<(unsigned)blocks, 128, 0, stream>>>(p);
    else if (yu) qconv_nchw_generic<false, true><<<(unsigned)blocks, 128, 0, stream>>>(p);
    else qconv_nchw_generic<false, false><<<(unsigned)blocks, 128, 0, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ZANT_E_CUDA, "launch of qconv_nchw_generic failed: %s", cudaGetErrorString(e));
    return ZANT_OK;
}
