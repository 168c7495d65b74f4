// Sample-sharded predict over several devices of one machine: one context, one stream, one arena
// and one host worker thread per device, no collective (samples are independent).  The reference
// bakes the batch into the generated predict() (src/codeGen/predict.zig:34-40, 317-336); this is
// the extension that splits one host batch across GPUs with zant_b200_shard_range and writes every
// device's result into its own slice of the caller's output buffer.
#include <cuda_runtime.h>

#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/zant_b200.h"
#include "context.cuh"
#include "status.hpp"

using namespace zb;

namespace {

struct MultiWorker {
    zant_ctx* ctx = nullptr;
    zant_plan* plan = nullptr;
    size_t batch = 0, in_bytes = 0, out_bytes = 0;   // of the plan's input / output tensors
    std::thread thread;
    std::mutex m;
    std::condition_variable cv;
    bool has_job = false, done = false, quit = false;
    const char* job_in = nullptr;
    char* job_out = nullptr;
    int32_t status = ZANT_OK;
    std::string message;
};

void worker_loop(MultiWorker* w) {
    cudaSetDevice(w->ctx->device);
    std::unique_lock<std::mutex> lock(w->m);
    while (true) {
        w->cv.wait(lock, [w] { return w->has_job || w->quit; });
        if (w->quit) return;
        w->has_job = false;
        lock.unlock();
        int32_t st = zant_b200_plan_run(w->plan, w->job_in, w->job_out);
        const int32_t sy = zant_b200_ctx_synchronize(w->ctx);      // also reports a device-side time-out
        if (st == ZANT_OK) st = sy;
        std::string msg = st == ZANT_OK ? std::string() : last_error_ref();
        lock.lock();
        w->status = st; w->message = std::move(msg); w->done = true;
        w->cv.notify_all();
    }
}

}  // namespace

struct zant_multi {
    std::vector<MultiWorker*> workers;
};

// "0,2,3" -> {0,2,3}; anything unparsable ends the list.
static std::vector<int32_t> devices_from_env() {
    std::vector<int32_t> out;
    const char* v = std::getenv("ZANT_B200_DEVICES");
    if (!v) return out;
    while (*v) {
        char* end = nullptr;
        const long d = std::strtol(v, &end, 10);
        if (end == v) break;
        out.push_back((int32_t)d);
        v = end;
        while (*v == ',' || *v == ' ') ++v;
    }
    return out;
}

extern "C" {

int32_t zant_b200_multi_create(const int32_t* devices, size_t n_devices, size_t arena_bytes, zant_multi** out) {
    if (!out) return fail(ZANT_E_NULL_POINTER, "out is NULL");
    *out = nullptr;
    std::vector<int32_t> list;
    if (devices && n_devices) list.assign(devices, devices + n_devices);
    else list = devices_from_env();
    if (list.empty()) {
        const int n = zant_b200_device_count();
        for (int d = 0; d < n; ++d) list.push_back(d);
    }
    if (list.empty()) return fail(ZANT_E_CUDA_UNAVAILABLE, "no CUDA device; there is no CPU fallback");
    zant_multi* m = new zant_multi();
    for (int32_t d : list) {
        zant_ctx* c = nullptr;
        const int32_t st = zant_b200_ctx_create(d, arena_bytes, &c);
        if (st != ZANT_OK) { zant_b200_multi_destroy(m); return st; }
        MultiWorker* w = new MultiWorker();
        w->ctx = c;
        m->workers.push_back(w);
        w->thread = std::thread(worker_loop, w);
    }
    *out = m;
    return ZANT_OK;
}

int32_t zant_b200_multi_destroy(zant_multi* m) {
    if (!m) return ZANT_OK;
    for (MultiWorker* w : m->workers) {
        {
            std::lock_guard<std::mutex> lock(w->m);
            w->quit = true;
        }
        w->cv.notify_all();
        if (w->thread.joinable()) w->thread.join();
        zant_b200_ctx_destroy(w->ctx);      // plans are the caller's: destroy them before the multi handle
        delete w;
    }
    delete m;
    return ZANT_OK;
}

size_t zant_b200_multi_size(zant_multi* m) { return m ? m->workers.size() : 0; }

zant_ctx* zant_b200_multi_ctx(zant_multi* m, size_t i) { return (m && i < m->workers.size()) ? m->workers[i]->ctx : nullptr; }

int32_t zant_b200_multi_set_plan(zant_multi* m, size_t i, zant_plan* plan) {
    if (!m || i >= m->workers.size()) return fail(ZANT_E_BAD_HANDLE, "multi handle is NULL or shard %zu does not exist", i);
    if (!plan || !plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan is NULL or not finalized");
    MultiWorker* w = m->workers[i];
    if (plan->ctx != w->ctx) return fail(ZANT_E_INVALID_INPUT, "the plan of shard %zu must be built on zant_b200_multi_ctx(multi, %zu)", i, i);
    const PlanTensor& ti = plan->t[plan->input];
    const PlanTensor& to = plan->t[plan->output];
    if (ti.shape.empty() || to.shape.empty() || ti.shape[0] == 0 || to.shape[0] != ti.shape[0])
        return fail(ZANT_E_INVALID_DIMENSIONS, "plan input and output must share a leading batch dimension");
    w->plan = plan; w->batch = ti.shape[0]; w->in_bytes = ti.bytes; w->out_bytes = to.bytes;
    return ZANT_OK;
}

int32_t zant_b200_predict_sharded(zant_multi* m, const void* host_in, void* host_out, size_t n_samples, int32_t* status_per_device) {
    if (!m || m->workers.empty()) return fail(ZANT_E_BAD_HANDLE, "multi handle is NULL");
    if (!host_in || !host_out) return fail(ZANT_E_NULL_POINTER, "input/output is NULL");
    const size_t world = m->workers.size();
    if (status_per_device) for (size_t i = 0; i < world; ++i) status_per_device[i] = ZANT_OK;
    // every shard's plan must hold exactly the samples zant_b200_shard_range gives it
    std::vector<size_t> begin(world), count(world);
    for (size_t i = 0; i < world; ++i) {
        ZB_TRY(zant_b200_shard_range(n_samples, world, i, &begin[i], &count[i]));
        MultiWorker* w = m->workers[i];
        if (count[i] == 0) continue;
        if (!w->plan) return fail(ZANT_E_BAD_HANDLE, "shard %zu has no plan", i);
        if (w->batch != count[i]) return fail(ZANT_E_INPUT_TENSOR_DIFFERENT_SIZE, "shard %zu: plan batch %zu, shard of %zu samples holds %zu", i, w->batch, n_samples, count[i]);
    }
    const char* in = static_cast<const char*>(host_in);
    char* outp = static_cast<char*>(host_out);
    size_t in_off = 0, out_off = 0;
    for (size_t i = 0; i < world; ++i) {
        MultiWorker* w = m->workers[i];
        if (count[i] == 0) continue;
        {
            std::lock_guard<std::mutex> lock(w->m);
            w->job_in = in + in_off; w->job_out = outp + out_off;
            w->done = false; w->has_job = true;
        }
        w->cv.notify_all();
        in_off += w->in_bytes; out_off += w->out_bytes;
    }
    int32_t first = ZANT_OK;
    for (size_t i = 0; i < world; ++i) {
        MultiWorker* w = m->workers[i];
        if (count[i] == 0) continue;
        std::unique_lock<std::mutex> lock(w->m);
        w->cv.wait(lock, [w] { return w->done; });
        if (status_per_device) status_per_device[i] = w->status;
        if (w->status != ZANT_OK && first == ZANT_OK) {
            first = w->status;
            last_error_ref() = "shard " + std::to_string(i) + ": " + w->message;
        }
    }
    return first;
}

}  // extern "C"
