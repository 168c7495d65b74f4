// Device context, staging of host buffers, launch bookkeeping.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <vector>

#include "status.hpp"

struct zant_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = true;
    char* arena = nullptr;        // staging arena for host-pointer calls and op workspaces
    size_t arena_bytes = 0;
    size_t arena_used = 0;
    size_t arena_limit = 0;       // 0 = the staging arena may grow on demand; else its hard cap in bytes
    uint64_t launches = 0;
    int sm_count = 148;
    int* status_word = nullptr;   // device int: kernels with bounded waits report here
    int tf32 = 0;                 // float contractions: 0 = the exact FP32 kernels, 1 = tensor cores (kind::tf32, single pass), 2 = tensor cores, split operands (3 x TF32)
};

namespace zb {

#define ZB_CUDA(expr)                                                                         \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            return zb::fail(ZANT_E_CUDA, "%s -> %s", #expr, cudaGetErrorString(_e));          \
    } while (0)

// Opt-in to more than 48 KiB of dynamic shared memory.  The attribute belongs to the function ON ONE DEVICE, so it is
// set once per device (a process may drive several: one worker thread per device, each with its own context).
#define ZB_SMEM_ATTR(ctx, kernel, bytes)                                                      \
    do {                                                                                      \
        static std::atomic<unsigned long long> zb_done_{0ull};                                \
        const unsigned long long zb_bit_ = 1ull << ((ctx)->device & 63);                      \
        if (!(zb_done_.load(std::memory_order_acquire) & zb_bit_)) {                          \
            ZB_CUDA(cudaFuncSetAttribute((kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes))); \
            zb_done_.fetch_or(zb_bit_, std::memory_order_release);                            \
        }                                                                                     \
    } while (0)

// Device allocations: an out-of-memory answer is the reference's MemError (src/Utils/errorHandler.zig:36-52).
#define ZB_ALLOC(ptr, bytes)                                                                  \
    do {                                                                                      \
        cudaError_t _e = zb::dev_malloc((void**)&(ptr), (bytes));                             \
        if (_e == cudaErrorMemoryAllocation) { cudaGetLastError(); return zb::fail(ZANT_E_MEM_ERROR, "device allocation of %zu bytes failed", (size_t)(bytes)); } \
        if (_e != cudaSuccess) return zb::fail(ZANT_E_CUDA, "cudaMalloc(%zu) -> %s", (size_t)(bytes), cudaGetErrorString(_e)); \
    } while (0)

#ifndef ZB_TRY
#define ZB_TRY(expr) do { int32_t _s = (expr); if (_s != ZANT_OK) return _s; } while (0)
#endif

inline int32_t check_launch(zant_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ZANT_E_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return ZANT_OK;
}

// Drains the stream and reads the device status word that kernels with bounded waits write when
// they give up; a non-zero value is reported once and cleared.
inline int32_t drain_and_check_status(zant_ctx* ctx) {
    int h = 0;
    ZB_CUDA(cudaMemcpyAsync(&h, ctx->status_word, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    ZB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (h != 0) {
        ZB_CUDA(cudaMemsetAsync(ctx->status_word, 0, sizeof(int), ctx->stream));
        return fail(ZANT_E_DEVICE_TIMEOUT, "a kernel gave up a bounded wait (device error %d)", h);
    }
    return ZANT_OK;
}

inline bool is_device_ptr(const void* p) {
    if (!p) return false;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Device memory that belongs to another GPU than `device`: a kernel of this context must not be
// handed such a pointer (without peer access it would take an illegal-address fault, which is sticky
// for the whole CUDA context).  Managed memory migrates and is accepted on every device.
inline bool is_foreign_device_ptr(const void* p, int device) {
    if (!p) return false;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice && a.device != device;
}

// Every device allocation of the library goes through here.  `alloc_failures_armed()` is the test
// hook behind zant_b200_debug_fail_alloc: while it is positive it counts allocations down and the
// one that reaches zero reports cudaErrorMemoryAllocation without touching the driver.
inline std::atomic<int>& alloc_failures_armed() {
    static std::atomic<int> n{0};
    return n;
}
inline cudaError_t dev_malloc(void** p, size_t bytes) {
    int armed = alloc_failures_armed().load();
    while (armed > 0) {
        if (alloc_failures_armed().compare_exchange_weak(armed, armed - 1)) {
            if (armed == 1) { *p = nullptr; return cudaErrorMemoryAllocation; }
            break;
        }
    }
    return cudaMalloc(p, bytes);
}

// Page-locked host memory (cudaHostAlloc / cudaHostRegister): copies to and from it are truly
// asynchronous, so calls that are handed such buffers do not wait for the stream.
inline bool is_pinned_host_ptr(const void* p) {
    if (!p) return false;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

constexpr size_t kArenaAlign = 256;
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline int32_t arena_reserve(zant_ctx* ctx, size_t need_total) {
    if (need_total <= ctx->arena_bytes) return ZANT_OK;
    if (ctx->arena_used != 0) return fail(ZANT_E_ARENA_EXHAUSTED, "arena of %zu bytes exhausted (need %zu)", ctx->arena_bytes, need_total);
    if (ctx->arena_limit && need_total > ctx->arena_limit)
        return fail(ZANT_E_ARENA_EXHAUSTED, "call needs %zu bytes of staging arena, the context's limit is %zu", need_total, ctx->arena_limit);
    ZB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->arena) ZB_CUDA(cudaFree(ctx->arena));
    ctx->arena = nullptr; ctx->arena_bytes = 0;
    size_t want = align_up(need_total + need_total / 4, 1 << 20);
    if (ctx->arena_limit && want > ctx->arena_limit) want = ctx->arena_limit;
    ZB_ALLOC(ctx->arena, want);
    ctx->arena_bytes = want;
    return ZANT_OK;
}

// Per-call staging: host inputs are copied into the arena, host outputs are copied back
// when the call finishes; device pointers pass through.  All buffers of one call must be
// declared (plan phase) before the first is materialised so the arena can grow once.
class Stager {
  public:
    explicit Stager(zant_ctx* c) : ctx_(c) {}
    ~Stager() { if (ctx_) ctx_->arena_used = 0; }

    struct Slot { const void* host_in; void* host_out; size_t bytes; size_t off; void* dev; bool staged; };

    int in(const void* p, size_t bytes) { return add(p, nullptr, bytes, true); }
    int out(void* p, size_t bytes) { return add(nullptr, p, bytes, false); }
    int scratch(size_t bytes) {
        Slot s{nullptr, nullptr, bytes, 0, nullptr, true};
        slots_.push_back(s);
        return (int)slots_.size() - 1;
    }

    // Allocates arena space for every staged slot and issues the H2D copies.
    int32_t commit() {
        if (foreign_) return fail(ZANT_E_INVALID_INPUT, "a device buffer belongs to another GPU than the context's device %d", ctx_->device);
        size_t total = 0;
        for (auto& s : slots_) if (s.staged) { s.off = total; total += align_up(s.bytes ? s.bytes : 1, kArenaAlign); }
        if (total) {
            int32_t st = arena_reserve(ctx_, total);
            if (st != ZANT_OK) return st;
            ctx_->arena_used = total;
        }
        for (auto& s : slots_) {
            if (!s.staged) continue;
            s.dev = ctx_->arena + s.off;
            if (s.host_in && s.bytes)
                ZB_CUDA(cudaMemcpyAsync(s.dev, s.host_in, s.bytes, cudaMemcpyHostToDevice, ctx_->stream));
        }
        return ZANT_OK;
    }

    template <typename T> T* ptr(int i) { return reinterpret_cast<T*>(slots_[i].dev); }

    // Copies staged outputs back and, if anything was staged, waits for the stream.
    int32_t finish() {
        bool any = false;
        for (auto& s : slots_) {
            if (!s.staged) continue;
            any = true;
            if (s.host_out && s.bytes)
                ZB_CUDA(cudaMemcpyAsync(s.host_out, s.dev, s.bytes, cudaMemcpyDeviceToHost, ctx_->stream));
        }
        if (any) {
            // the call waits anyway: also pick up the status word that a bounded device-side wait writes
            // when it gives up, so that the time-out is reported by the call that suffered it
            const int32_t st = drain_and_check_status(ctx_);
            ctx_->arena_used = 0;
            return st;
        }
        return ZANT_OK;
    }

  private:
    int add(const void* pin, void* pout, size_t bytes, bool is_in) {
        const void* p = is_in ? pin : pout;
        Slot s{nullptr, nullptr, bytes, 0, nullptr, false};
        if (p == nullptr) { s.dev = nullptr; }
        else if (is_device_ptr(p)) { s.dev = const_cast<void*>(p); foreign_ = foreign_ || is_foreign_device_ptr(p, ctx_->device); }
        else { s.staged = true; s.host_in = pin; s.host_out = pout; }
        slots_.push_back(s);
        return (int)slots_.size() - 1;
    }
    zant_ctx* ctx_;
    std::vector<Slot> slots_;
    bool foreign_ = false;
};

inline int grid_for(size_t work_items, int block, int sm_count, int waves = 8) {
    size_t blocks = (work_items + block - 1) / block;
    const size_t cap = (size_t)sm_count * waves;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return (int)blocks;
}

}  // namespace zb
