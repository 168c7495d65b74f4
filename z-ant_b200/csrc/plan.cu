// Plan: the run-time form of a generated predict() — graph tensors at fixed offsets of one
// cudaMalloc'd arena, constants uploaded once, nodes launched in insertion order.
// (src/codeGen/predict.zig:23-70 emits the straight-line op calls this replays;
//  :110-142, :265-272 is the one-static-array-per-tensor memory plan mirrored here.)
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <algorithm>
#include <cmath>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "../../include/zant_b200.h"
#include "context.cuh"
#include "geometry.hpp"
#include "ops.cuh"
#include "fused_cnn.cuh"
#include "tc_gemm.cuh"
#include "tc_conv_generic.cuh"
#include "tc_conv_nchw.cuh"
#include "tc_pw_nchw.cuh"
#include "dwconv_q8.cuh"
#include "smallc_conv_q8.cuh"
#include "tc_conv_nhwc.cuh"
#include "tc_gemm_tf32.cuh"
#include "status.hpp"

using namespace zb;

struct PlanTensor {
    int32_t dtype = ZANT_F32;
    std::vector<size_t> shape;
    size_t bytes = 0;
    bool is_const = false;
    std::vector<char> host;     // initializer bytes (kept until finalize)
    size_t offset = 0;          // arena offset
    void* arena_ptr = nullptr;  // address inside the plan's arena
    void* bound = nullptr;      // caller's device buffer bound for the current run (input/output)
    int alias = -1;             // Reshape output: shares the buffer of this tensor
    bool elided = false;        // interior of a fused chain: never materialised, no arena space
};

struct PlanNode {
    int32_t op = 0;
    std::vector<int> in, out;
    zant_node_attrs a{};
};

struct zant_plan {
    zant_ctx* ctx = nullptr;
    std::vector<PlanTensor> t;
    std::vector<PlanNode> nodes;
    std::vector<std::vector<char>> aux_host;   // derived constants (multipliers, tables)
    std::vector<size_t> aux_off;
    std::vector<size_t> scratch_bytes;         // internal buffers of fused steps (private layouts)
    std::vector<size_t> scratch_off;
    int input = -1, output = -1;
    bool finalized = false;
    char* arena = nullptr;
    size_t arena_bytes = 0;
    std::vector<std::function<int32_t()>> steps;
    std::vector<std::string> step_names;
    std::vector<double> step_macs, step_bytes;   // algorithmic work of each step: multiply-accumulates, bytes crossing the step's boundary
    int launches_per_run = 0;
    bool profiling = false;
    cudaGraphExec_t graph_exec = nullptr;   // replay of all steps on arena buffers
    std::vector<cudaEvent_t> prof_events;   // pool, reused between reads
    size_t prof_used = 0;                   // events recorded since the last read

    void* ptr(int id) const {
        int r = id;
        while (t[r].alias >= 0) r = t[r].alias;
        return t[r].bound ? t[r].bound : t[r].arena_ptr;
    }
    template <typename T> T* p(int id) const { return id < 0 ? nullptr : reinterpret_cast<T*>(ptr(id)); }
    void* aux(int id) const { return arena + aux_off[id]; }
    void* scratch(int id) const { return arena + scratch_off[id]; }
    int add_scratch(size_t bytes) { scratch_bytes.push_back(bytes); return (int)scratch_bytes.size() - 1; }
    // One buffer for the im2col matrices of all tensor-core steps: steps run one after another on
    // one stream, so they can share it; it is as large as the largest request.
    // float activation that the fusion pass asks the next Conv step to apply, and the tensor that step writes instead of its own
    int pending_fact = 0; float pending_slope = 0.0f; int pending_y = -1; bool pending_used = false;
    int im2col_scratch = -1;
    int shared_im2col_scratch(size_t bytes) {
        if (im2col_scratch < 0) im2col_scratch = add_scratch(bytes);
        else scratch_bytes[im2col_scratch] = std::max(scratch_bytes[im2col_scratch], bytes);
        return im2col_scratch;
    }
    int add_aux(const void* data, size_t bytes) {
        aux_host.emplace_back((const char*)data, (const char*)data + bytes);
        return (int)aux_host.size() - 1;
    }
};

namespace {

const char* kAutoPadNames[] = {"NOTSET", "SAME_UPPER", "SAME_LOWER", "VALID"};

int32_t need_inputs(const PlanNode& n, size_t lo, size_t hi, const char* name) {
    if (n.in.size() < lo || n.in.size() > hi) return fail(ZANT_E_INVALID_INPUT, "%s takes %zu..%zu inputs, got %zu", name, lo, hi, n.in.size());
    if (n.out.size() != 1) return fail(ZANT_E_INVALID_INPUT, "%s produces one output", name);
    return ZANT_OK;
}

int opt_in(const PlanNode& n, size_t i) { return i < n.in.size() ? n.in[i] : -1; }

int32_t want_dtype(const zant_plan* pl, int id, int32_t dt, const char* what) {
    if (id >= 0 && pl->t[id].dtype != dt) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "%s: tensor %d has dtype %d, expected %d", what, id, pl->t[id].dtype, dt);
    return ZANT_OK;
}

// Table for a unary function between two quantized tensors:
//   lut[code] = sat(rne(f(float(q - zp_in) * s_in) / s_out) + zp_out)
template <typename F>
void build_unary_lut(int32_t dtype, float s_in, int zp_in, float s_out, int zp_out, F f, uint8_t lut[256]) {
    for (int code = 0; code < 256; ++code) {
        const int q = dtype == ZANT_U8 ? code : (int)(int8_t)(uint8_t)code;
        volatile float x = (float)(q - zp_in) * s_in;
        volatile float a = f((float)x);
        volatile float v = a / s_out;
        float c = std::fmin(std::fmax((float)v, -512.0f), 511.0f);
        int t = (int)std::nearbyintf(c) + zp_out;
        const int lo = dtype == ZANT_U8 ? 0 : -128, hi = dtype == ZANT_U8 ? 255 : 127;
        t = std::min(std::max(t, lo), hi);
        lut[code] = (uint8_t)t;
    }
}

// Table of a Relu / LeakyRelu / Clip node between two quantized tensors of type `dt`.
void activation_lut(const PlanNode& n, int32_t dt, uint8_t lut[256]) {
    const zant_node_attrs& a = n.a;
    const float p0 = a.alpha, p1 = a.beta;
    if (n.op == ZANT_OP_RELU) build_unary_lut(dt, a.x_scale, a.x_zp, a.y_scale, a.y_zp, [](float v) { return v > 0.0f ? v : 0.0f; }, lut);
    else if (n.op == ZANT_OP_LEAKY_RELU) build_unary_lut(dt, a.x_scale, a.x_zp, a.y_scale, a.y_zp, [p0](float v) { volatile float s = p0 * v; return v <= 0.0f ? (float)s : v; }, lut);
    else build_unary_lut(dt, a.x_scale, a.x_zp, a.y_scale, a.y_zp, [p0, p1](float v) { return std::fmin(std::fmax(v, p0), p1); }, lut);
}

}  // namespace

extern "C" {

int32_t zant_b200_plan_create(zant_ctx* ctx, zant_plan** out) {
    if (!out) return fail(ZANT_E_NULL_POINTER, "out is NULL");
    *out = nullptr;
    if (!ctx) return fail(ZANT_E_CUDA_UNAVAILABLE, "no context; there is no CPU fallback");
    zant_plan* p = new zant_plan();
    p->ctx = ctx;
    *out = p;
    return ZANT_OK;
}

int32_t zant_b200_plan_destroy(zant_plan* plan) {
    if (!plan) return ZANT_OK;
    cudaSetDevice(plan->ctx->device);
    cudaStreamSynchronize(plan->ctx->stream);
    if (plan->graph_exec) cudaGraphExecDestroy(plan->graph_exec);
    if (plan->arena) cudaFree(plan->arena);
    for (cudaEvent_t e : plan->prof_events) cudaEventDestroy(e);
    cudaGetLastError();
    delete plan;
    return ZANT_OK;
}

int32_t zant_b200_plan_tensor(zant_plan* plan, int32_t dtype, const size_t* shape, size_t rank, const void* const_data, int32_t* id) {
    if (!plan) return fail(ZANT_E_BAD_HANDLE, "plan is NULL");
    if (plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan already finalized");
    if (!id || (rank && !shape)) return fail(ZANT_E_NULL_POINTER, "id/shape is NULL");
    if (!dtype_valid(dtype)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "dtype %d", dtype);
    if (rank > 8) return fail(ZANT_E_UNSUPPORTED_DIMENSION, "rank %zu", rank);
    PlanTensor t;
    t.dtype = dtype;
    t.shape.assign(shape, shape + rank);
    t.bytes = numel(shape, rank) * dtype_size(dtype);
    if (const_data) {
        t.is_const = true;
        t.host.assign((const char*)const_data, (const char*)const_data + t.bytes);
    }
    plan->t.push_back(std::move(t));
    *id = (int32_t)plan->t.size() - 1;
    return ZANT_OK;
}

int32_t zant_b200_plan_node(zant_plan* plan, int32_t op, const int32_t* inputs, size_t n_inputs,
                            const int32_t* outputs, size_t n_outputs, const zant_node_attrs* attrs) {
    if (!plan) return fail(ZANT_E_BAD_HANDLE, "plan is NULL");
    if (plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan already finalized");
    if ((n_inputs && !inputs) || (n_outputs && !outputs)) return fail(ZANT_E_NULL_POINTER, "inputs/outputs is NULL");
    PlanNode n;
    n.op = op;
    const int nt = (int)plan->t.size();
    for (size_t i = 0; i < n_inputs; ++i) {
        if (inputs[i] < -1 || inputs[i] >= nt) return fail(ZANT_E_INVALID_INPUT, "input %zu: unknown tensor id %d", i, inputs[i]);
        n.in.push_back(inputs[i]);
    }
    for (size_t i = 0; i < n_outputs; ++i) {
        if (outputs[i] < 0 || outputs[i] >= nt) return fail(ZANT_E_INVALID_INPUT, "output %zu: unknown tensor id %d", i, outputs[i]);
        if (plan->t[outputs[i]].is_const) return fail(ZANT_E_INVALID_INPUT, "output %zu is an initializer", i);
        n.out.push_back(outputs[i]);
    }
    if (attrs) n.a = *attrs;
    plan->nodes.push_back(std::move(n));
    return ZANT_OK;
}

static int32_t build_node(zant_plan* pl, size_t node_index, int32_t fuse);
static int32_t build_node_impl(zant_plan* pl, size_t node_index, int32_t fuse);
static int32_t try_fuse(zant_plan* pl, size_t node_index, size_t& consumed);
static int32_t try_fuse_small_cnn(zant_plan* pl, size_t node_index, size_t& consumed);
static int32_t try_fuse_qconv_group(zant_plan* pl, size_t node_index, size_t& consumed);
static int32_t try_fuse_fconv_group(zant_plan* pl, size_t node_index, size_t& consumed);

// Multiply-accumulates of one node (contractions only; everything else counts as 0).
static double node_macs(const zant_plan* pl, const PlanNode& n) {
    auto shape = [&](int id) -> const std::vector<size_t>& { return pl->t[id].shape; };
    auto count = [&](int id) { double c = 1; for (size_t d : shape(id)) c *= (double)d; return c; };
    switch (n.op) {
        case ZANT_OP_CONV:
        case ZANT_OP_QLINEAR_CONV: {
            if (n.in.size() < 2 || n.out.empty() || shape(n.in[1]).size() != 4) return 0;
            const auto& w = shape(n.in[1]);
            return count(n.out[0]) * (double)w[1] * (double)w[2] * (double)w[3];
        }
        case ZANT_OP_MATMUL:
        case ZANT_OP_QLINEAR_MATMUL:
        case ZANT_OP_GEMM: {
            if (n.in.size() < 2 || n.out.empty() || shape(n.in[0]).size() < 2) return 0;
            const auto& a = shape(n.in[0]);
            const size_t k = (n.op == ZANT_OP_GEMM && n.a.trans_a) ? a[a.size() - 2] : a[a.size() - 1];
            return count(n.out[0]) * (double)k;
        }
        default: return 0;
    }
}

// Cost of the steps that cover nodes [first, first + count): MACs of the nodes; bytes = every tensor that is read
// from outside the group (initializers included) or written by it and still materialised, each counted once.
static void record_step_cost(zant_plan* pl, size_t first_step, size_t first, size_t count) {
    double macs = 0, bytes = 0;
    std::vector<char> produced(pl->t.size(), 0), seen(pl->t.size(), 0);
    auto root = [&](int id) { while (pl->t[id].alias >= 0) id = pl->t[id].alias; return id; };
    for (size_t i = first; i < first + count; ++i) for (int o : pl->nodes[i].out) produced[root(o)] = 1;
    for (size_t i = first; i < first + count; ++i) {
        const PlanNode& n = pl->nodes[i];
        macs += node_macs(pl, n);
        if (n.op == ZANT_OP_RESHAPE) continue;
        for (int id : n.in) {
            if (id < 0) continue;
            const int r = root(id);
            if (!produced[r] && !seen[r]) { seen[r] = 1; bytes += (double)pl->t[id].bytes; }
        }
        for (int o : n.out) {
            const int r = root(o);
            if (!pl->t[r].elided && !seen[r]) { seen[r] = 1; bytes += (double)pl->t[o].bytes; }
        }
    }
    pl->step_macs.resize(pl->steps.size(), 0.0);
    pl->step_bytes.resize(pl->steps.size(), 0.0);
    if (pl->steps.size() > first_step) {       // a group may emit several steps: the work is booked on its last one
        pl->step_macs.back() = macs;
        pl->step_bytes.back() = bytes;
    }
}

int32_t zant_b200_plan_finalize(zant_plan* plan, int32_t input_id, int32_t output_id, int32_t fuse) {
    if (!plan) return fail(ZANT_E_BAD_HANDLE, "plan is NULL");
    if (plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan already finalized");
    const int nt = (int)plan->t.size();
    if (input_id < 0 || input_id >= nt || output_id < 0 || output_id >= nt) return fail(ZANT_E_INVALID_INPUT, "input/output id out of range");
    plan->input = input_id; plan->output = output_id;
    zant_ctx* ctx = plan->ctx;
    ZB_CUDA(cudaSetDevice(ctx->device));

    // 1. validate nodes, derive constants, record launch closures
    plan->steps.clear(); plan->step_names.clear(); plan->step_macs.clear(); plan->step_bytes.clear();
    size_t i = 0;
    while (i < plan->nodes.size()) {
        size_t consumed = 0;
        if (fuse) {
            int32_t st = try_fuse(plan, i, consumed);
            if (st != ZANT_OK) return st;
        }
        if (consumed == 0) {
            int32_t st = build_node(plan, i, fuse);
            if (st != ZANT_OK) return st;
            consumed = 1;
        }
        i += consumed;
    }

    // 2. arena layout: every non-aliased tensor and every derived constant at a fixed offset
    size_t off = 0;
    for (auto& t : plan->t) {
        if (t.alias >= 0 || t.elided) continue;
        t.offset = off;
        off += align_up(t.bytes ? t.bytes : 1, kArenaAlign);
    }
    plan->aux_off.resize(plan->aux_host.size());
    for (size_t a = 0; a < plan->aux_host.size(); ++a) {
        plan->aux_off[a] = off;
        off += align_up(plan->aux_host[a].size() ? plan->aux_host[a].size() : 1, kArenaAlign);
    }
    plan->scratch_off.resize(plan->scratch_bytes.size());
    for (size_t a = 0; a < plan->scratch_bytes.size(); ++a) {
        plan->scratch_off[a] = off;
        off += align_up(plan->scratch_bytes[a] ? plan->scratch_bytes[a] : 1, kArenaAlign);
    }
    plan->arena_bytes = off;
    ZB_ALLOC(plan->arena, off);
    for (auto& t : plan->t) {
        if (t.alias >= 0 || t.elided) continue;
        t.arena_ptr = plan->arena + t.offset;
        if (t.is_const && t.bytes) ZB_CUDA(cudaMemcpyAsync(t.arena_ptr, t.host.data(), t.bytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    for (size_t a = 0; a < plan->aux_host.size(); ++a)
        if (!plan->aux_host[a].empty())
            ZB_CUDA(cudaMemcpyAsync(plan->arena + plan->aux_off[a], plan->aux_host[a].data(), plan->aux_host[a].size(), cudaMemcpyHostToDevice, ctx->stream));
    ZB_CUDA(cudaStreamSynchronize(ctx->stream));
    for (auto& t : plan->t) { t.host.clear(); t.host.shrink_to_fit(); }

    // 3. one dry count of launches
    plan->finalized = true;
    const uint64_t before = ctx->launches;
    for (auto& s : plan->steps) { int32_t st = s(); if (st != ZANT_OK) { plan->finalized = false; return st; } }
    ZB_CUDA(cudaStreamSynchronize(ctx->stream));
    plan->launches_per_run = (int)(ctx->launches - before);
    ctx->launches = before;
    log_line("zant_b200 plan: %zu tensors, %zu nodes, %zu steps, %d launches, arena %zu bytes", plan->t.size(), plan->nodes.size(), plan->steps.size(), plan->launches_per_run, plan->arena_bytes);
    return ZANT_OK;
}

int32_t zant_b200_plan_run(zant_plan* plan, const void* input, void* output) {
    if (!plan || !plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan is NULL or not finalized");
    if (!input || !output) return fail(ZANT_E_NULL_POINTER, "input/output is NULL");
    zant_ctx* ctx = plan->ctx;
    ZB_CUDA(cudaSetDevice(ctx->device));
    PlanTensor& ti = plan->t[plan->input];
    PlanTensor& to = plan->t[plan->output];
    int out_root = plan->output;
    while (plan->t[out_root].alias >= 0) out_root = plan->t[out_root].alias;
    PlanTensor& tor = plan->t[out_root];
    const bool in_dev = is_device_ptr(input), out_dev = is_device_ptr(output);
    if (is_foreign_device_ptr(input, ctx->device) || is_foreign_device_ptr(output, ctx->device))
        return fail(ZANT_E_INVALID_INPUT, "input/output is device memory of another GPU than the plan's device %d", ctx->device);
    if (plan->graph_exec && !plan->profiling) {
        // replay: everything runs on the arena's own buffers
        ZB_CUDA(cudaMemcpyAsync(ti.arena_ptr, input, ti.bytes, in_dev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream));
        ZB_CUDA(cudaGraphLaunch(plan->graph_exec, ctx->stream));
        ctx->launches += (uint64_t)plan->launches_per_run;
        ZB_CUDA(cudaMemcpyAsync(output, tor.arena_ptr, to.bytes, out_dev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, ctx->stream));
        if (out_dev || (is_pinned_host_ptr(output) && (in_dev || is_pinned_host_ptr(input)))) return ZANT_OK;
        return drain_and_check_status(ctx);
    }
    ti.bound = in_dev ? const_cast<void*>(input) : nullptr;
    tor.bound = out_dev ? output : nullptr;
    if (!in_dev) ZB_CUDA(cudaMemcpyAsync(ti.arena_ptr, input, ti.bytes, cudaMemcpyHostToDevice, ctx->stream));
    auto mark = [&]() -> int32_t {
        if (plan->prof_used == plan->prof_events.size()) {
            cudaEvent_t e;
            ZB_CUDA(cudaEventCreate(&e));
            plan->prof_events.push_back(e);
        }
        ZB_CUDA(cudaEventRecord(plan->prof_events[plan->prof_used++], ctx->stream));
        return ZANT_OK;
    };
    for (size_t s = 0; s < plan->steps.size(); ++s) {
        if (plan->profiling) { int32_t st = mark(); if (st != ZANT_OK) return st; }
        int32_t st = plan->steps[s]();
        if (st != ZANT_OK) { ti.bound = nullptr; tor.bound = nullptr; return st; }
    }
    if (plan->profiling) { int32_t st = mark(); if (st != ZANT_OK) return st; }
    if (!out_dev) {
        ZB_CUDA(cudaMemcpyAsync(output, tor.arena_ptr, to.bytes, cudaMemcpyDeviceToHost, ctx->stream));
        ti.bound = nullptr; tor.bound = nullptr;
        // Pinned host buffers on both sides: the whole run stays asynchronous on the stream (the
        // caller overlaps it with other contexts and calls zant_b200_ctx_synchronize).  Pageable
        // buffers: wait, so that the result is in place when the call returns.
        if (is_pinned_host_ptr(output) && (in_dev || is_pinned_host_ptr(input))) return ZANT_OK;
        return drain_and_check_status(ctx);
    }
    ti.bound = nullptr; tor.bound = nullptr;
    return ZANT_OK;
}

int32_t zant_b200_plan_use_graph(zant_plan* plan, int32_t enable) {
    if (!plan || !plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan is NULL or not finalized");
    zant_ctx* ctx = plan->ctx;
    ZB_CUDA(cudaSetDevice(ctx->device));
    ZB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (plan->graph_exec) { cudaGraphExecDestroy(plan->graph_exec); plan->graph_exec = nullptr; }
    if (!enable) return ZANT_OK;
    // every step has run at least once (the dry run of finalize), so one-time function attributes are set
    plan->t[plan->input].bound = nullptr;
    {
        int r = plan->output;
        while (plan->t[r].alias >= 0) r = plan->t[r].alias;
        plan->t[r].bound = nullptr;
    }
    const uint64_t before = ctx->launches;
    ZB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    int32_t st = ZANT_OK;
    for (auto& step : plan->steps) { st = step(); if (st != ZANT_OK) break; }
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    ctx->launches = before;
    if (st != ZANT_OK) { if (graph) cudaGraphDestroy(graph); return st; }
    if (e != cudaSuccess || !graph) { cudaGetLastError(); return fail(ZANT_E_CUDA, "stream capture failed: %s", cudaGetErrorString(e)); }
    const cudaError_t ei = cudaGraphInstantiate(&plan->graph_exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ei != cudaSuccess) { plan->graph_exec = nullptr; cudaGetLastError(); return fail(ZANT_E_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(ei)); }
    return ZANT_OK;
}

size_t zant_b200_plan_arena_bytes(zant_plan* plan) { return plan ? plan->arena_bytes : 0; }
int32_t zant_b200_plan_launches_per_run(zant_plan* plan) { return plan ? plan->launches_per_run : 0; }
void* zant_b200_plan_tensor_ptr(zant_plan* plan, int32_t id) {
    if (!plan || !plan->finalized || id < 0 || id >= (int)plan->t.size()) return nullptr;
    return plan->ptr(id);
}

int32_t zant_b200_plan_step_count(zant_plan* plan) { return (plan && plan->finalized) ? (int32_t)plan->steps.size() : 0; }
const char* zant_b200_plan_step_name(zant_plan* plan, int32_t step) {
    if (!plan || step < 0 || step >= (int32_t)plan->step_names.size()) return "";
    return plan->step_names[step].c_str();
}

int32_t zant_b200_plan_step_cost(zant_plan* plan, int32_t step, double* macs, double* bytes) {
    if (!plan || !plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan is NULL or not finalized");
    if (step < 0 || step >= (int32_t)plan->steps.size()) return fail(ZANT_E_INVALID_INPUT, "step %d of %zu", step, plan->steps.size());
    if (macs) *macs = step < (int32_t)plan->step_macs.size() ? plan->step_macs[step] : 0.0;
    if (bytes) *bytes = step < (int32_t)plan->step_bytes.size() ? plan->step_bytes[step] : 0.0;
    return ZANT_OK;
}

int32_t zant_b200_plan_profile(zant_plan* plan, int32_t enable) {
    if (!plan || !plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan is NULL or not finalized");
    plan->profiling = enable != 0;
    plan->prof_used = 0;
    return ZANT_OK;
}

int32_t zant_b200_plan_profile_read(zant_plan* plan, float* sum_ms, int32_t* runs) {
    if (!plan || !plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan is NULL or not finalized");
    if (!sum_ms || !runs) return fail(ZANT_E_NULL_POINTER, "sum_ms/runs is NULL");
    ZB_CUDA(cudaSetDevice(plan->ctx->device));
    ZB_CUDA(cudaStreamSynchronize(plan->ctx->stream));
    const size_t per_run = plan->steps.size() + 1;
    const size_t n_runs = plan->prof_used / per_run;
    for (size_t r = 0; r < n_runs; ++r)
        for (size_t s = 0; s + 1 < per_run; ++s) {
            float ms = 0.0f;
            ZB_CUDA(cudaEventElapsedTime(&ms, plan->prof_events[r * per_run + s], plan->prof_events[r * per_run + s + 1]));
            sum_ms[s] += ms;
        }
    *runs = (int32_t)n_runs;
    plan->prof_used = 0;
    return ZANT_OK;
}

int32_t zant_b200_plan_read_tensor(zant_plan* plan, int32_t id, void* host_dst) {
    if (!plan || !plan->finalized) return fail(ZANT_E_BAD_HANDLE, "plan is NULL or not finalized");
    if (id < 0 || id >= (int)plan->t.size()) return fail(ZANT_E_INVALID_INPUT, "tensor id %d", id);
    if (!host_dst) return fail(ZANT_E_NULL_POINTER, "host_dst is NULL");
    {
        int r = id;
        while (plan->t[r].alias >= 0) r = plan->t[r].alias;
        if (plan->t[r].elided) return fail(ZANT_E_UNSUPPORTED, "tensor %d is interior to a fused chain and is not materialised", id);
    }
    ZB_CUDA(cudaSetDevice(plan->ctx->device));
    ZB_CUDA(cudaStreamSynchronize(plan->ctx->stream));
    ZB_CUDA(cudaMemcpy(host_dst, plan->ptr(id), plan->t[id].bytes, cudaMemcpyDeviceToHost));
    return ZANT_OK;
}

}  // extern "C"

// --------------------------------------------------------------------------------------------
// QLinearConv, alone or as the head of a fused group.  `fz` carries what the fusion pass found behind the node:
// an activation override (a Relu that keeps scale and zero point), a 256-entry table (LeakyRelu, Clip, a Relu
// that changes scale) applied to the finished codes, the tensor the step writes instead of the node's own
// output, and a 2x2 / stride-2 MaxPool that the implicit-GEMM kernel can apply in its epilogue.
// --------------------------------------------------------------------------------------------
struct QConvFusion {
    int activation = -1;     // >= 0: replaces the node's own activation attribute
    int lut_aux = -1;        // aux id of the table, -1 = none
    int y_act = -1;          // tensor written when the pool is not fused (-1: the node's output)
    int y_pool = -1;         // pooled tensor; >= 0 asks for the fused pool
    bool pool_done = false;  // out: the step writes y_pool
};

static int32_t build_qconv(zant_plan* pl, const PlanNode& n, QConvFusion& fz) {
    const zant_node_attrs& a = n.a;
    zant_ctx* ctx = pl->ctx;
    auto T = [&](int id) -> const PlanTensor& { return pl->t[id]; };
    ZB_TRY(need_inputs(n, 3, 5, "QLinearConv"));
    const int x = n.in[0], w = n.in[1], ws = n.in[2], wz = opt_in(n, 3), b = opt_in(n, 4), y0 = n.out[0];
    if (x < 0 || w < 0 || ws < 0) return fail(ZANT_E_INVALID_INPUT, "QLinearConv needs x, w, w_scale");
    ZB_TRY(want_dtype(pl, w, ZANT_I8, "QLinearConv w")); ZB_TRY(want_dtype(pl, ws, ZANT_F32, "QLinearConv w_scale"));
    ZB_TRY(want_dtype(pl, wz, ZANT_I32, "QLinearConv w_zp")); ZB_TRY(want_dtype(pl, b, ZANT_I32, "QLinearConv bias"));
    const int32_t xd = T(x).dtype, yd = T(y0).dtype;
    if ((xd != ZANT_I8 && xd != ZANT_U8) || (yd != ZANT_I8 && yd != ZANT_U8)) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearConv x/y dtype");
    ZB_TRY(check_zero_point(xd, a.x_zp, "QLinearConv x"));
    if (!T(w).is_const || !T(ws).is_const || (wz >= 0 && !T(wz).is_const)) return fail(ZANT_E_UNSUPPORTED, "QLinearConv weights and scales must be initializers");
    ConvGeom g;
    if (a.channels_last) {
        // the geometry is that of the NCHW operator on the permuted shapes
        if (T(x).shape.size() != 4 || T(y0).shape.size() != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "channels-last QLinearConv takes rank-4 tensors");
        const size_t xs[4] = {T(x).shape[0], T(x).shape[3], T(x).shape[1], T(x).shape[2]}, ys[4] = {T(y0).shape[0], T(y0).shape[3], T(y0).shape[1], T(y0).shape[2]};
        ZB_TRY(conv_resolve_onnx(xs, 4, T(w).shape.data(), T(w).shape.size(), ys, 4,
                                 a.strides, a.n_strides, a.pads, a.n_pads, a.dilations, a.n_dilations, a.group, a.auto_pad < 0 ? 0 : a.auto_pad, g));
    } else {
        ZB_TRY(conv_resolve_onnx(T(x).shape.data(), T(x).shape.size(), T(w).shape.data(), T(w).shape.size(), T(y0).shape.data(), T(y0).shape.size(),
                                 a.strides, a.n_strides, a.pads, a.n_pads, a.dilations, a.n_dilations, a.group, a.auto_pad < 0 ? 0 : a.auto_pad, g));
    }
    const size_t nws = numel(T(ws).shape.data(), T(ws).shape.size());
    if (nws != 1 && nws != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearConv w_scale size");
    if (b >= 0 && numel(T(b).shape.data(), T(b).shape.size()) != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearConv bias size");
    std::vector<float> mult;
    requant_multipliers(a.x_scale, (const float*)T(ws).host.data(), nws, a.y_scale, (size_t)g.M, mult);
    std::vector<int32_t> wzv((size_t)g.M, 0);
    if (wz >= 0) {
        const size_t nwz = numel(T(wz).shape.data(), T(wz).shape.size());
        if (nwz != 1 && nwz != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearConv w_zp size");
        for (int m = 0; m < g.M; ++m) wzv[m] = ((const int32_t*)T(wz).host.data())[nwz == 1 ? 0 : m];
    }
    const int xzp = a.x_zp;
    const Requant rq0{a.y_scale, a.y_zp, fz.activation >= 0 ? fz.activation : a.activation};
    const int lut_aux = fz.lut_aux;
    // the requantisation parameters with the table's device address, resolved at launch time (the arena exists by then)
    auto rq_of = [pl, rq0, lut_aux]() { Requant r = rq0; r.lut = lut_aux >= 0 ? (const uint8_t*)pl->aux(lut_aux) : nullptr; return r; };
    bool wz_zero = true;
    for (int32_t v : wzv) wz_zero = wz_zero && v == 0;
    const bool const_bias = b < 0 || T(b).is_const;
    const int y = fz.y_act >= 0 ? fz.y_act : y0;          // written unless the pool is fused too
    const std::string tail = std::string(fz.activation >= 0 ? "+Relu" : "") + (lut_aux >= 0 ? "+ActivationLut" : "");
    auto push = [&](const std::string& name, std::function<int32_t()> fn) { pl->steps.push_back(std::move(fn)); pl->step_names.push_back(name); };
    fz.pool_done = false;

    if (a.channels_last) {
        TcConvPlan ncp;
        if (!const_bias || !tc_conv_nhwc_plan(g, wz_zero, xzp, ncp)) return fail(ZANT_E_UNSUPPORTED, "shape not taken by the channels-last QLinearConv kernel");
        std::vector<int8_t> w_blk; std::vector<float> mp; std::vector<int32_t> bp;
        tc_conv_nhwc_prepare(ncp, (const int8_t*)T(w).host.data(), mult.data(), b >= 0 ? (const int32_t*)T(b).host.data() : nullptr, xzp, w_blk, mp, bp);
        const int aw = pl->add_aux(w_blk.data(), w_blk.size()), am = pl->add_aux(mp.data(), mp.size() * 4), ab = pl->add_aux(bp.data(), bp.size() * 4);
        const double max_product = tc_conv_max_product(mp, bp, (long long)g.Cg * g.KH * g.KW);
        push("QLinearConv(tc-nhwc)" + tail, [=]() {
            if (!tc_conv_ptr_ok(pl->ptr(x)) || !tc_conv_ptr_ok(pl->ptr(y))) return fail(ZANT_E_INVALID_INPUT, "channels-last QLinearConv buffers must be 16-byte aligned");
            return tc_conv_nhwc_run(ctx, ncp, pl->ptr(x), xd == ZANT_U8, (const int8_t*)pl->aux(aw), (const float*)pl->aux(am),
                                    (const int32_t*)pl->aux(ab), pl->ptr(y), yd == ZANT_U8, rq_of(), max_product);
        });
        return ZANT_OK;
    }
    PwConvPlan pwp;
    const bool stem = const_bias && pw_stem_plan(g, wz_zero, xzp, ctx->sm_count, pwp);
    if (stem || (const_bias && pw_conv_plan(g, wz_zero, ctx->sm_count, pwp))) {
        // 1x1: filters on the accumulator lanes, activations straight from NCHW as the MN-major operand; 3x3 stems: the same
        // kernel on patches written in shared memory
        std::vector<int8_t> w_blk; std::vector<int32_t> bf;
        pw_conv_prepare(pwp, (const int8_t*)T(w).host.data(), b >= 0 ? (const int32_t*)T(b).host.data() : nullptr, xzp, w_blk, bf);
        bool finite = true;
        for (float f : mult) finite = finite && std::isfinite(f);
        const int aw = pl->add_aux(w_blk.data(), w_blk.size()), am = pl->add_aux(mult.data(), mult.size() * 4), ab = pl->add_aux(bf.data(), bf.size() * 4);
        std::vector<int32_t> caps;
        const bool capped = finite && yd == ZANT_I8 && rq0.y_zp == 0 && requant_relu_caps(mult.data(), mult.size(), rq0.act, lean_six(rq0.y_scale), caps);
        const int ac = capped ? pl->add_aux(caps.data(), caps.size() * 4) : -1;
        push(std::string(stem ? "QLinearConv(tc-stem)" : "QLinearConv(tc-pointwise)") + tail, [=]() {
            if (!pw_conv_ptr_ok(pl->ptr(x), pl->ptr(y))) return fail(ZANT_E_INVALID_INPUT, "pointwise QLinearConv buffers must be 16-byte (input) and 32-byte (output) aligned");
            return pw_conv_run(ctx, pwp, pl->ptr(x), xd == ZANT_U8, (const int8_t*)pl->aux(aw), (const float*)pl->aux(am),
                               (const int32_t*)pl->aux(ab), pl->ptr(y), yd == ZANT_U8, rq_of(), finite, ac >= 0 ? (const int32_t*)pl->aux(ac) : nullptr);
        });
        return ZANT_OK;
    }
    if (const_bias && qconv_smallc_eligible(g, wz_zero)) {
        // 3x3 on at most four input channels (network stems); arena tensors are 256-byte aligned
        std::vector<uint32_t> wfrag; std::vector<int32_t> bf;
        qconv_smallc_prepare(g, (const int8_t*)T(w).host.data(), b >= 0 ? (const int32_t*)T(b).host.data() : nullptr, xzp, wfrag, bf);
        const int aw = pl->add_aux(wfrag.data(), wfrag.size() * 4), am = pl->add_aux(mult.data(), mult.size() * 4), ab = pl->add_aux(bf.data(), bf.size() * 4);
        const double max_product = tc_conv_max_product(mult, bf, (long long)g.C * 9);
        push("QLinearConv(small-c)" + tail, [=]() {
            if (!qconv_smallc_ptr_ok(pl->ptr(x))) return fail(ZANT_E_INVALID_INPUT, "QLinearConv input buffer must be 4-byte aligned");
            return run_qconv_smallc(ctx, g, pl->ptr(x), xd == ZANT_U8, xzp, (const uint32_t*)pl->aux(aw), (const float*)pl->aux(am),
                                    (const int32_t*)pl->aux(ab), pl->ptr(y), yd == ZANT_U8, rq_of(), max_product);
        });
        return ZANT_OK;
    }
    TcConvPlan tcp;
    if (const_bias && (long long)g.N * g.OH * g.OW >= 256) {
        // implicit GEMM from NCHW (stride 1): weights blocked once here, one launch per run; with a fused pool the
        // epilogue writes the pooled tensor only.  Arena tensors are 256-byte aligned; a caller-bound input that is
        // not 16-byte aligned is refused at run time.
        const bool pooled = fz.y_pool >= 0 && tc_conv_plan(g, wz_zero, tcp, true);
        if (pooled || tc_conv_plan(g, wz_zero, tcp, false)) {
            std::vector<int8_t> w_blk; std::vector<float> mp; std::vector<int32_t> bp;
            tc_conv_prepare(tcp, (const int8_t*)T(w).host.data(), mult.data(), b >= 0 ? (const int32_t*)T(b).host.data() : nullptr, xzp, w_blk, mp, bp);
            const int aw = pl->add_aux(w_blk.data(), w_blk.size()), am = pl->add_aux(mp.data(), mp.size() * 4), ab = pl->add_aux(bp.data(), bp.size() * 4);
            const double max_product = tc_conv_max_product(mp, bp, (long long)g.Cg * g.KH * g.KW);
            const int yw = pooled ? fz.y_pool : y;
            fz.pool_done = pooled;
            push("QLinearConv(tc-implicit)" + tail + (pooled ? "+MaxPool" : ""), [=]() {
                if (!tc_conv_ptr_ok(pl->ptr(x))) return fail(ZANT_E_INVALID_INPUT, "QLinearConv input buffer must be 16-byte aligned");
                return tc_conv_run(ctx, tcp, pl->ptr(x), xd == ZANT_U8, xzp, (const int8_t*)pl->aux(aw), (const float*)pl->aux(am),
                                   (const int32_t*)pl->aux(ab), pl->ptr(yw), yd == ZANT_U8, rq_of(), max_product);
            });
            return ZANT_OK;
        }
    }
    if (const_bias && qdwconv_eligible(g, wz_zero)) {
        // depthwise 3x3: one HBM-bound pass; arena tensors are 256-byte aligned
        std::vector<uint32_t> wrow; std::vector<int32_t> bf;
        qdwconv_prepare(g, (const int8_t*)T(w).host.data(), b >= 0 ? (const int32_t*)T(b).host.data() : nullptr, xzp, wrow, bf);
        bool finite = true;
        for (float f : mult) finite = finite && std::isfinite(f);
        const int aw = pl->add_aux(wrow.data(), wrow.size() * 4), am = pl->add_aux(mult.data(), mult.size() * 4), ab = pl->add_aux(bf.data(), bf.size() * 4);
        std::vector<int32_t> caps;
        const bool capped = finite && yd == ZANT_I8 && rq0.y_zp == 0 && requant_relu_caps(mult.data(), mult.size(), rq0.act, lean_six(rq0.y_scale), caps);
        const int ac = capped ? pl->add_aux(caps.data(), caps.size() * 4) : -1;
        push("QLinearConv(depthwise)" + tail, [=]() {
            if (!qdwconv_ptr_ok(pl->ptr(x)) || !qdwconv_ptr_ok(pl->ptr(y))) return fail(ZANT_E_INVALID_INPUT, "depthwise QLinearConv buffers must be 4-byte aligned");
            return run_qdwconv(ctx, g, pl->ptr(x), xd == ZANT_U8, xzp, (const uint32_t*)pl->aux(aw), (const float*)pl->aux(am),
                               (const int32_t*)pl->aux(ab), pl->ptr(y), yd == ZANT_U8, rq_of(), finite, ac >= 0 ? (const int32_t*)pl->aux(ac) : nullptr);
        });
        return ZANT_OK;
    }
    if (qconv_tc_eligible(g, wz_zero) && const_bias) {
        // tensor-core path: weights re-blocked once here, im2col + tcgen05 GEMM per run
        auto prep = std::make_shared<QGemmPrep>();
        qconv_gemm_prepare(g, (const int8_t*)T(w).host.data(), mult.data(), b >= 0 ? (const int32_t*)T(b).host.data() : nullptr, xzp, *prep);
        const int aw = pl->add_aux(prep->w_blk.data(), prep->w_blk.size()), am = pl->add_aux(prep->mult.data(), prep->mult.size() * 4);
        const int ab = pl->add_aux(prep->bias.data(), prep->bias.size() * 4);
        const int sa = pl->shared_im2col_scratch(qgemm_a_bytes((size_t)g.N * g.OH * g.OW, *prep));
        prep->w_blk.clear(); prep->w_blk.shrink_to_fit();
        push("QLinearConv(tc)" + tail, [=]() {
            return run_qconv_tc(ctx, g, pl->ptr(x), xd == ZANT_U8, xzp, *prep, (const int8_t*)pl->aux(aw), (const float*)pl->aux(am),
                                (const int32_t*)pl->aux(ab), (uint8_t*)pl->scratch(sa), pl->ptr(y), yd == ZANT_U8, rq_of());
        });
        return ZANT_OK;
    }
    const int am = pl->add_aux(mult.data(), mult.size() * 4), az = pl->add_aux(wzv.data(), wzv.size() * 4);
    push("QLinearConv" + tail, [=]() {
        QConvArgs q{};
        q.x = pl->ptr(x); q.w = pl->p<int8_t>(w); q.y = pl->ptr(y);
        q.mult = (const float*)pl->aux(am); q.w_zp = (const int32_t*)pl->aux(az); q.bias = pl->p<int32_t>(b);
        q.x_zp = xzp; q.rq = rq_of(); q.g = g;
        return run_qconv_generic(ctx, q, xd, yd);
    });
    return ZANT_OK;
}

// --------------------------------------------------------------------------------------------
// One node -> one (or a few) kernel launches, using the same resolvers as the single-op ABI.
// --------------------------------------------------------------------------------------------
static int32_t build_node(zant_plan* pl, size_t node_index, int32_t fuse) {
    const size_t first_step = pl->steps.size();
    ZB_TRY(build_node_impl(pl, node_index, fuse));
    record_step_cost(pl, first_step, node_index, 1);
    return ZANT_OK;
}

static int32_t build_node_impl(zant_plan* pl, size_t node_index, int32_t /*fuse*/) {
    const PlanNode& n = pl->nodes[node_index];
    const zant_node_attrs& a = n.a;
    zant_ctx* ctx = pl->ctx;
    auto T = [&](int id) -> const PlanTensor& { return pl->t[id]; };
    auto push = [&](const char* name, std::function<int32_t()> fn) { pl->steps.push_back(std::move(fn)); pl->step_names.push_back(name); };

    switch (n.op) {
        case ZANT_OP_CONV: {
            ZB_TRY(need_inputs(n, 2, 3, "Conv"));
            const int x = n.in[0], w = n.in[1], b = opt_in(n, 2), y = n.out[0];
            ZB_TRY(want_dtype(pl, x, ZANT_F32, "Conv")); ZB_TRY(want_dtype(pl, w, ZANT_F32, "Conv")); ZB_TRY(want_dtype(pl, y, ZANT_F32, "Conv"));
            ConvGeom g;
            const char* ap = (a.auto_pad >= 0 && a.auto_pad <= 3) ? kAutoPadNames[a.auto_pad] : nullptr;
            ZB_TRY(conv_resolve_ref(T(x).shape.data(), T(x).shape.size(), T(w).shape.data(), T(w).shape.size(),
                                    T(y).shape.data(), T(y).shape.size(), a.strides, a.n_strides,
                                    a.n_pads ? a.pads : nullptr, a.n_pads, a.n_dilations ? a.dilations : nullptr, a.n_dilations,
                                    a.group, ap, ap ? std::strlen(ap) : 0, g));
            if (b >= 0 && numel(T(b).shape.data(), T(b).shape.size()) != (size_t)g.M) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "Conv bias size");
            if (ctx->tf32 && T(w).is_const && (b < 0 || T(b).is_const) && g.M <= 2048 && (long long)g.N * g.OH * g.OW >= 128) {
                // tensor-core float path: weights blocked once here; im2col gather + tcgen05 kind::tf32 GEMM per run, with the
                // activation the fusion pass found behind the node in the epilogue
                auto prep = std::make_shared<TfGemmPrep>();
                const int K = g.C * g.KH * g.KW;
                tf_gemm_prepare((const float*)T(w).host.data(), g.M, K, K, 1, b >= 0 ? (const float*)T(b).host.data() : nullptr, *prep, (long long)g.N * g.OH * g.OW, ctx->tf32 == 2);
                tf_conv_table(g, *prep);
                const int aw = pl->add_aux(prep->w_blk.data(), prep->w_blk.size() * 4), ab = pl->add_aux(prep->bias.data(), prep->bias.size() * 4);
                const int at = pl->add_aux(prep->ktab.data(), prep->ktab.size() * 4);
                const int sa = pl->shared_im2col_scratch(tf_gemm_a_bytes((size_t)g.N * g.OH * g.OW, *prep));
                prep->w_blk.clear(); prep->w_blk.shrink_to_fit();
                const int fact = pl->pending_fact; const float fslope = pl->pending_slope;
                const int yw = pl->pending_y >= 0 ? pl->pending_y : y;
                push(fact == FACT_NONE ? "Conv(tf32)" : (fact == FACT_RELU ? "Conv(tf32)+Relu" : "Conv(tf32)+LeakyRelu"), [=]() {
                    return run_conv_tf32(ctx, g, pl->p<float>(x), *prep, (const float*)pl->aux(aw), (const float*)pl->aux(ab), (const int32_t*)pl->aux(at), (float*)pl->scratch(sa), fact, fslope, pl->p<float>(yw));
                });
                pl->pending_used = true;
                return ZANT_OK;
            }
            push("Conv", [=]() { return run_conv_f32(ctx, g, pl->p<float>(x), pl->p<float>(w), pl->p<float>(b), pl->p<float>(y)); });
            return ZANT_OK;
        }
        case ZANT_OP_MATMUL: {
            ZB_TRY(need_inputs(n, 2, 2, "MatMul"));
            const int x = n.in[0], w = n.in[1], y = n.out[0];
            MatGeom g;
            ZB_TRY(matmul_check(T(x).shape.data(), T(x).shape.size(), T(w).shape.data(), T(w).shape.size(), T(y).shape.data(), T(y).shape.size(), g));
            if (ctx->tf32 && T(w).is_const && T(w).dtype == ZANT_F32 && g.N <= 2048 && g.M >= 128 && g.K <= 0x7fffffffULL && g.M <= 0x7fffffffULL) {
                auto prep = std::make_shared<TfGemmPrep>();
                tf_gemm_prepare((const float*)T(w).host.data(), (int)g.N, (int)g.K, 1, (long long)g.N, nullptr, *prep, (long long)g.M, ctx->tf32 == 2);
                const int aw = pl->add_aux(prep->w_blk.data(), prep->w_blk.size() * 4), ab = pl->add_aux(prep->bias.data(), prep->bias.size() * 4);
                const int sa = pl->shared_im2col_scratch(tf_gemm_a_bytes(g.M, *prep));
                prep->w_blk.clear(); prep->w_blk.shrink_to_fit();
                const MatGeom gg = g;
                push("MatMul(tf32)", [=]() {
                    return run_matmul_tf32(ctx, pl->p<float>(x), (long long)gg.M, (int)gg.K, (long long)gg.K, 1, *prep, (const float*)pl->aux(aw), (const float*)pl->aux(ab),
                                           (float*)pl->scratch(sa), FACT_NONE, 0.0f, pl->p<float>(y));
                });
                return ZANT_OK;
            }
            push("MatMul", [=]() { return run_matmul_f32(ctx, g, pl->p<float>(x), pl->p<float>(w), pl->p<float>(y)); });
            return ZANT_OK;
        }
        case ZANT_OP_GEMM: {
            ZB_TRY(need_inputs(n, 2, 3, "Gemm"));
            const int x = n.in[0], w = n.in[1], c = opt_in(n, 2), y = n.out[0];
            GemmGeom g;
            ZB_TRY(gemm_check_lean(T(x).shape.data(), T(x).shape.size(), T(w).shape.data(), T(w).shape.size(),
                              c >= 0 ? T(c).shape.data() : nullptr, c >= 0 ? T(c).shape.size() : 0, c >= 0,
                              a.trans_a != 0, a.trans_b != 0, a.beta, T(y).shape.data(), T(y).shape.size(), g));
            const float alpha = a.alpha, beta = a.beta; const bool ta = a.trans_a != 0, tb = a.trans_b != 0;
            {
                // tensor-core float path for the fully-connected form: Y = A B' + row vector C (alpha = beta = 1)
                const bool c_row = c < 0 || (T(c).is_const && beta == 1.0f && g.c_mode != 0 && g.c_rows == 1 && g.c_cols == g.cols && numel(T(c).shape.data(), T(c).shape.size()) == g.cols);
                if (ctx->tf32 && !ta && alpha == 1.0f && T(w).is_const && c_row && g.batch == 1 && g.cols <= 2048 && g.rows >= 128 && g.K <= 0x7fffffffULL && g.rows <= 0x7fffffffULL) {
                    auto prep = std::make_shared<TfGemmPrep>();
                    tf_gemm_prepare((const float*)T(w).host.data(), (int)g.cols, (int)g.K, tb ? (long long)g.K : 1, tb ? 1 : (long long)g.cols,
                                    c >= 0 ? (const float*)T(c).host.data() : nullptr, *prep, (long long)g.rows, ctx->tf32 == 2);
                    const int aw = pl->add_aux(prep->w_blk.data(), prep->w_blk.size() * 4), ab = pl->add_aux(prep->bias.data(), prep->bias.size() * 4);
                    const int sa = pl->shared_im2col_scratch(tf_gemm_a_bytes(g.rows, *prep));
                    prep->w_blk.clear(); prep->w_blk.shrink_to_fit();
                    const GemmGeom gg = g;
                    push("Gemm(tf32)", [=]() {
                        return run_matmul_tf32(ctx, pl->p<float>(x), (long long)gg.rows, (int)gg.K, (long long)gg.K, 1, *prep, (const float*)pl->aux(aw), (const float*)pl->aux(ab),
                                               (float*)pl->scratch(sa), FACT_NONE, 0.0f, pl->p<float>(y));
                    });
                    return ZANT_OK;
                }
            }
            push("Gemm", [=]() { return run_gemm_f32(ctx, g, pl->p<float>(x), pl->p<float>(w), pl->p<float>(c), alpha, beta, ta, tb, pl->p<float>(y)); });
            return ZANT_OK;
        }
        case ZANT_OP_MAXPOOL: {
            ZB_TRY(need_inputs(n, 1, 1, "MaxPool"));
            const int x = n.in[0], y = n.out[0];
            PoolGeom g;
            const size_t ones[2] = {1, 1};
            ZB_TRY(pool_resolve(T(x).shape.data(), T(x).shape.size(), T(y).shape.data(), T(y).shape.size(), a.kernel_shape, 2,
                                a.n_strides ? a.strides : ones, 2, a.n_dilations ? a.dilations : ones, 2, a.pads, a.n_pads, a.auto_pad < 0 ? 0 : a.auto_pad, g));
            const int32_t dt = T(x).dtype;
            if (dt != T(y).dtype) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "MaxPool dtype mismatch");
            if (dt == ZANT_F32) push("MaxPool", [=]() { return run_maxpool<float>(ctx, g, pl->p<float>(x), pl->p<float>(y)); });
            else if (dt == ZANT_I8) push("MaxPool", [=]() { return run_maxpool<int8_t>(ctx, g, pl->p<int8_t>(x), pl->p<int8_t>(y)); });
            else if (dt == ZANT_U8) push("MaxPool", [=]() { return run_maxpool<uint8_t>(ctx, g, pl->p<uint8_t>(x), pl->p<uint8_t>(y)); });
            else return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "MaxPool on int32");
            return ZANT_OK;
        }
        case ZANT_OP_TRANSPOSE:
        case ZANT_OP_SLICE: {
            ZB_TRY(need_inputs(n, 1, 1, "Transpose/Slice"));
            const int x = n.in[0], y = n.out[0];
            if (T(x).dtype != T(y).dtype) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "Transpose/Slice dtype mismatch");
            StridedMap m;
            const std::vector<size_t>& xs = T(x).shape; const std::vector<size_t>& ys = T(y).shape;
            if (n.op == ZANT_OP_TRANSPOSE) {
                size_t perm[8];
                if (a.n_perm > 8) return fail(ZANT_E_INVALID_PERMUTATION, "perm holds %zu entries", a.n_perm);
                for (size_t i = 0; i < a.n_perm; ++i) perm[i] = a.perm[i] < 0 ? (size_t)-1 : (size_t)a.perm[i];
                ZB_TRY(transpose_resolve(xs.data(), xs.size(), a.n_perm ? perm : nullptr, a.n_perm, ys.data(), ys.size(), m));
            } else {
                if (a.n_slice > 8) return fail(ZANT_E_INVALID_SLICE_INDICES, "%zu slice entries", a.n_slice);
                size_t od[8];
                ZB_TRY(slice_resolve(xs.data(), xs.size(), a.slice_starts, a.slice_ends, a.n_slice, a.slice_has_axes ? a.slice_axes : nullptr,
                                     a.slice_has_steps ? a.slice_steps : nullptr, od, &m));
                if (ys.size() != xs.size()) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "Slice output rank");
                for (size_t d = 0; d < xs.size(); ++d) if (ys[d] != od[d]) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "Slice output dim %zu", d);
            }
            const size_t esz = dtype_size(T(x).dtype);
            push(n.op == ZANT_OP_TRANSPOSE ? "Transpose" : "Slice", [=]() { return run_strided_copy(ctx, esz, pl->ptr(x), pl->ptr(y), m); });
            return ZANT_OK;
        }
        case ZANT_OP_GATHER: {
            ZB_TRY(need_inputs(n, 2, 2, "Gather"));
            const int x = n.in[0], ind = n.in[1], y = n.out[0];
            if (T(x).dtype != T(y).dtype) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "Gather dtype mismatch");
            ZB_TRY(want_dtype(pl, ind, ZANT_I32, "Gather indices"));
            if (!T(ind).is_const) return fail(ZANT_E_UNSUPPORTED, "Gather indices must be an initializer");
            const size_t ni = numel(T(ind).shape.data(), T(ind).shape.size());
            std::vector<size_t> idx(ni);
            for (size_t i = 0; i < ni; ++i) {
                const int32_t v = ((const int32_t*)T(ind).host.data())[i];
                idx[i] = v < 0 ? (size_t)-1 : (size_t)v;      // a negative index is out of bounds, as for the reference's usize
            }
            GatherGeom g;
            ZB_TRY(gather_resolve(T(x).shape.data(), T(x).shape.size(), idx.data(), T(ind).shape.data(), T(ind).shape.size(), a.axis,
                                  T(y).shape.data(), T(y).shape.size(), g));
            const size_t esz = dtype_size(T(x).dtype);
            push("Gather", [=]() { return run_gather(ctx, esz, pl->ptr(x), pl->p<int32_t>(ind), pl->ptr(y), g); });
            return ZANT_OK;
        }
        case ZANT_OP_SIGMOID:
        case ZANT_OP_TANH:
        case ZANT_OP_CEIL: {
            ZB_TRY(need_inputs(n, 1, 1, "unary"));
            const int x = n.in[0], y = n.out[0];
            ZB_TRY(want_dtype(pl, x, ZANT_F32, "unary")); ZB_TRY(want_dtype(pl, y, ZANT_F32, "unary"));
            const size_t cnt = numel(T(x).shape.data(), T(x).shape.size());
            if (cnt != numel(T(y).shape.data(), T(y).shape.size())) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "unary sizes differ");
            if (n.op == ZANT_OP_SIGMOID) push("Sigmoid", [=]() { return run_unary_f32(ctx, pl->p<float>(x), pl->p<float>(y), cnt, SigmoidOp{}, "sigmoid_f32"); });
            else if (n.op == ZANT_OP_TANH) push("Tanh", [=]() { return run_unary_f32(ctx, pl->p<float>(x), pl->p<float>(y), cnt, TanhOp{}, "tanh_f32"); });
            else push("Ceil", [=]() { return run_unary_f32(ctx, pl->p<float>(x), pl->p<float>(y), cnt, CeilOp{}, "ceil_f32"); });
            return ZANT_OK;
        }
        case ZANT_OP_SOFTMAX: {
            ZB_TRY(need_inputs(n, 1, 1, "Softmax"));
            const int x = n.in[0], y = n.out[0];
            ZB_TRY(want_dtype(pl, x, ZANT_F32, "Softmax")); ZB_TRY(want_dtype(pl, y, ZANT_F32, "Softmax"));
            if (T(x).shape.size() != 2) return fail(ZANT_E_INVALID_DIMENSIONS, "Softmax takes a 2-D tensor");
            if (T(y).shape != T(x).shape) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "Softmax shapes differ");
            const size_t rows = T(x).shape[0], cols = T(x).shape[1];
            push("Softmax", [=]() { return run_softmax_f32(ctx, pl->p<float>(x), pl->p<float>(y), rows, cols); });
            return ZANT_OK;
        }
        case ZANT_OP_MUL:
        case ZANT_OP_DIV: {
            ZB_TRY(need_inputs(n, 2, 2, "Mul/Div"));
            const int x = n.in[0], w = n.in[1], y = n.out[0];
            ZB_TRY(want_dtype(pl, x, ZANT_F32, "Mul/Div")); ZB_TRY(want_dtype(pl, w, ZANT_F32, "Mul/Div")); ZB_TRY(want_dtype(pl, y, ZANT_F32, "Mul/Div"));
            const size_t cnt = numel(T(x).shape.data(), T(x).shape.size());
            if (cnt != numel(T(w).shape.data(), T(w).shape.size())) return fail(ZANT_E_MISMATCHED_SHAPE, "Mul/Div operands differ in size");
            if (cnt != numel(T(y).shape.data(), T(y).shape.size())) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "Mul/Div output size");
            const bool divide = n.op == ZANT_OP_DIV;
            push(divide ? "Div" : "Mul", [=]() { return run_binary_same_f32(ctx, pl->p<float>(x), pl->p<float>(w), pl->p<float>(y), cnt, divide); });
            return ZANT_OK;
        }
        case ZANT_OP_RELU:
        case ZANT_OP_LEAKY_RELU:
        case ZANT_OP_CLIP: {
            ZB_TRY(need_inputs(n, 1, 1, "activation"));
            const int x = n.in[0], y = n.out[0];
            const size_t cnt = numel(T(x).shape.data(), T(x).shape.size());
            if (cnt != numel(T(y).shape.data(), T(y).shape.size())) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "activation sizes differ");
            const int32_t dt = T(x).dtype;
            if (dt != T(y).dtype) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "activation dtype mismatch");
            const float p0 = a.alpha, p1 = a.beta;
            if (dt == ZANT_F32) {
                if (n.op == ZANT_OP_RELU) push("Relu", [=]() { return run_unary_f32(ctx, pl->p<float>(x), pl->p<float>(y), cnt, ReluOp{}, "relu_f32"); });
                else if (n.op == ZANT_OP_LEAKY_RELU) push("LeakyRelu", [=]() { return run_unary_f32(ctx, pl->p<float>(x), pl->p<float>(y), cnt, LeakyOp{p0}, "leaky_relu_f32"); });
                else push("Clip", [=]() { return run_unary_f32(ctx, pl->p<float>(x), pl->p<float>(y), cnt, ClipOp{p0, p1}, "clip_f32"); });
                return ZANT_OK;
            }
            if (dt == ZANT_I32) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "activation on int32");
            // Quantized tensors: dequantise, activate, requantise through a 256-entry table.
            uint8_t lut[256];
            activation_lut(n, dt, lut);
            const int aux = pl->add_aux(lut, 256);
            push("ActivationLut", [=]() { return run_lut(ctx, pl->p<char>(x), pl->p<char>(y), cnt, (const uint8_t*)pl->aux(aux)); });
            return ZANT_OK;
        }
        case ZANT_OP_ADD: {
            ZB_TRY(need_inputs(n, 2, 2, "Add"));
            const int x = n.in[0], w = n.in[1], y = n.out[0];
            ZB_TRY(want_dtype(pl, x, ZANT_F32, "Add")); ZB_TRY(want_dtype(pl, w, ZANT_F32, "Add")); ZB_TRY(want_dtype(pl, y, ZANT_F32, "Add"));
            BcastGeom g;
            ZB_TRY(bcast_resolve(T(x).shape.data(), T(x).shape.size(), T(w).shape.data(), T(w).shape.size(), T(y).shape.data(), T(y).shape.size(), g));
            push("Add", [=]() { return run_add_f32(ctx, g, pl->p<float>(x), pl->p<float>(w), pl->p<float>(y)); });
            return ZANT_OK;
        }
        case ZANT_OP_CONCAT: {
            if (n.in.empty() || n.out.size() != 1) return fail(ZANT_E_EMPTY_TENSOR_LIST, "Concat needs inputs and one output");
            const int y = n.out[0];
            std::vector<const size_t*> shapes; std::vector<size_t> ranks;
            for (int id : n.in) {
                if (id < 0) return fail(ZANT_E_INVALID_INPUT, "Concat input missing");
                if (T(id).dtype != T(y).dtype) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "Concat dtype mismatch");
                shapes.push_back(T(id).shape.data()); ranks.push_back(T(id).shape.size());
            }
            ConcatGeom g; size_t os[8];
            ZB_TRY(concat_resolve(shapes.data(), ranks.data(), n.in.size(), a.axis, os, g));
            if (T(y).shape.size() != g.rank) return fail(ZANT_E_MISMATCHED_RANK, "Concat output rank");
            for (size_t d = 0; d < g.rank; ++d) if (T(y).shape[d] != os[d]) return fail(ZANT_E_MISMATCHED_SHAPE, "Concat output dim %zu", d);
            const size_t esz = dtype_size(T(y).dtype);
            const std::vector<int> ins = n.in;
            push("Concat", [=]() {
                std::vector<const void*> ptrs(ins.size());
                for (size_t i = 0; i < ins.size(); ++i) ptrs[i] = pl->ptr(ins[i]);
                return run_concat(ctx, g, esz, ptrs.data(), pl->ptr(y));
            });
            return ZANT_OK;
        }
        case ZANT_OP_RESIZE: {
            ZB_TRY(need_inputs(n, 1, 1, "Resize"));
            const int x = n.in[0], y = n.out[0];
            const size_t r = T(x).shape.size();
            if (r == 0 || r > 4 || a.n_scales != r) return fail(ZANT_E_INVALID_INPUT, "Resize scales length != rank");
            if (T(x).dtype != T(y).dtype) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "Resize dtype mismatch");
            std::vector<size_t> os(r);
            ZB_TRY(resize_output_shape(T(x).shape.data(), r, a.scales, a.n_scales, nullptr, 0, os.data()));
            if (T(y).shape != os) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "Resize output shape");
            std::vector<int32_t> table, axis_offset;
            resize_index_table(T(x).shape.data(), os.data(), r, a.coord_mode, table, axis_offset);
            const int aux = pl->add_aux(table.data(), table.size() * 4);
            const std::vector<size_t> xs = T(x).shape;
            const size_t esz = dtype_size(T(x).dtype);
            push("Resize", [=]() { return run_resize(ctx, esz, pl->ptr(x), pl->ptr(y), (const int32_t*)pl->aux(aux), xs.data(), os.data(), r, axis_offset); });
            return ZANT_OK;
        }
        case ZANT_OP_REDUCE_MEAN: {
            ZB_TRY(need_inputs(n, 1, 1, "ReduceMean"));
            const int x = n.in[0], y = n.out[0];
            ZB_TRY(want_dtype(pl, x, ZANT_F32, "ReduceMean")); ZB_TRY(want_dtype(pl, y, ZANT_F32, "ReduceMean"));
            ReduceGeom g;
            ZB_TRY(reduce_resolve(T(x).shape.data(), T(x).shape.size(), T(y).shape.data(), T(y).shape.size(), a.n_axes ? a.axes : nullptr, a.n_axes, a.noop_with_empty_axes != 0, g));
            push("ReduceMean", [=]() { return run_reduce_mean_f32(ctx, g, pl->p<float>(x), pl->p<float>(y)); });
            return ZANT_OK;
        }
        case ZANT_OP_RESHAPE: {
            ZB_TRY(need_inputs(n, 1, 1, "Reshape"));
            const int x = n.in[0], y = n.out[0];
            if (T(x).dtype != T(y).dtype) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "Reshape dtype mismatch");
            if (numel(T(x).shape.data(), T(x).shape.size()) != numel(T(y).shape.data(), T(y).shape.size()))
                return fail(ZANT_E_INPUT_ARRAY_WRONG_SIZE, "Reshape changes the element count");
            // Row-major order is preserved, so the output is a view: no kernel, no copy.
            pl->t[y].alias = x;
            return ZANT_OK;
        }
        case ZANT_OP_QUANTIZE_LINEAR: {
            ZB_TRY(need_inputs(n, 1, 1, "QuantizeLinear"));
            const int x = n.in[0], y = n.out[0];
            ZB_TRY(want_dtype(pl, x, ZANT_F32, "QuantizeLinear"));
            const int32_t dt = T(y).dtype;
            if (dt != ZANT_I8 && dt != ZANT_U8) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QuantizeLinear output dtype");
            const size_t cnt = numel(T(x).shape.data(), T(x).shape.size());
            if (cnt != numel(T(y).shape.data(), T(y).shape.size())) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "QuantizeLinear sizes differ");
            const float sc = a.y_scale; const int zp = a.y_zp;
            push("QuantizeLinear", [=]() { return run_quantize(ctx, pl->p<float>(x), pl->ptr(y), cnt, sc, zp, dt); });
            return ZANT_OK;
        }
        case ZANT_OP_DEQUANTIZE_LINEAR: {
            ZB_TRY(need_inputs(n, 1, 1, "DequantizeLinear"));
            const int x = n.in[0], y = n.out[0];
            ZB_TRY(want_dtype(pl, y, ZANT_F32, "DequantizeLinear"));
            const int32_t dt = T(x).dtype;
            if (dt == ZANT_F32) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "DequantizeLinear input dtype");
            const size_t cnt = numel(T(x).shape.data(), T(x).shape.size());
            if (cnt != numel(T(y).shape.data(), T(y).shape.size())) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "DequantizeLinear sizes differ");
            const float sc = a.x_scale; const int zp = a.x_zp;
            push("DequantizeLinear", [=]() { return run_dequantize(ctx, dt, pl->ptr(x), pl->p<float>(y), cnt, sc, zp); });
            return ZANT_OK;
        }
        case ZANT_OP_QLINEAR_CONV: {
            QConvFusion none;
            return build_qconv(pl, n, none);
        }
        case ZANT_OP_QLINEAR_MATMUL: {
            ZB_TRY(need_inputs(n, 3, 5, "QLinearMatMul"));
            const int x = n.in[0], w = n.in[1], ws = n.in[2], wz = opt_in(n, 3), b = opt_in(n, 4), y = n.out[0];
            if (x < 0 || w < 0 || ws < 0) return fail(ZANT_E_INVALID_INPUT, "QLinearMatMul needs a, b, b_scale");
            ZB_TRY(want_dtype(pl, w, ZANT_I8, "QLinearMatMul b")); ZB_TRY(want_dtype(pl, ws, ZANT_F32, "QLinearMatMul b_scale"));
            ZB_TRY(want_dtype(pl, wz, ZANT_I32, "QLinearMatMul b_zp")); ZB_TRY(want_dtype(pl, b, ZANT_I32, "QLinearMatMul bias"));
            const int32_t xd = T(x).dtype, yd = T(y).dtype;
            if (xd != ZANT_I8 && xd != ZANT_U8) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearMatMul a dtype");
            ZB_TRY(check_zero_point(xd, a.x_zp, "QLinearMatMul a"));
            if (yd == ZANT_F32) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearMatMul y dtype");
            if (!T(w).is_const || !T(ws).is_const || (wz >= 0 && !T(wz).is_const)) return fail(ZANT_E_UNSUPPORTED, "QLinearMatMul weights and scales must be initializers");
            if (T(x).shape.size() != 2 || T(w).shape.size() != 2 || T(y).shape.size() != 2) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearMatMul takes 2-D operands");
            const size_t M = T(x).shape[0], K = T(x).shape[1], N = T(w).shape[1];
            if (T(w).shape[0] != K || M * N == 0 || K == 0) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearMatMul inner dims");
            if (T(y).shape[0] != M || T(y).shape[1] != N) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "QLinearMatMul output shape");
            const size_t nws = numel(T(ws).shape.data(), T(ws).shape.size());
            if (nws != 1 && nws != N) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearMatMul b_scale size");
            if (b >= 0 && numel(T(b).shape.data(), T(b).shape.size()) != N) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearMatMul bias size");
            std::vector<float> mult;
            requant_multipliers(a.x_scale, (const float*)T(ws).host.data(), nws, a.y_scale, N, mult);
            std::vector<int32_t> bz(N, 0);
            if (wz >= 0) {
                const size_t nwz = numel(T(wz).shape.data(), T(wz).shape.size());
                if (nwz != 1 && nwz != N) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "QLinearMatMul b_zp size");
                for (size_t j = 0; j < N; ++j) bz[j] = ((const int32_t*)T(wz).host.data())[nwz == 1 ? 0 : j];
            }
            const int xzp = a.x_zp; const Requant rq{a.y_scale, a.y_zp, a.activation};
            bool bz_zero = true;
            for (int32_t v : bz) bz_zero = bz_zero && v == 0;
            if (M <= 0x7fffffffULL && N <= 0x7fffffffULL && K <= 0x7fffffffULL) {
                ConvGeom g{};   // a matrix product is a 1x1 convolution over M "images" of one pixel
                g.N = (int)M; g.C = (int)K; g.H = g.W = 1; g.M = (int)N; g.Cg = (int)K; g.KH = g.KW = 1;
                g.sh = g.sw = g.dh = g.dw = 1; g.OH = g.OW = 1; g.G = 1;
                if (yd != ZANT_I32 && qconv_tc_eligible(g, bz_zero) && (b < 0 || T(b).is_const)) {
                    std::vector<int8_t> bt(K * N);
                    const int8_t* bw = (const int8_t*)T(w).host.data();
                    for (size_t k = 0; k < K; ++k) for (size_t j = 0; j < N; ++j) bt[j * K + k] = bw[k * N + j];
                    auto prep = std::make_shared<QGemmPrep>();
                    qgemm_prepare(bt.data(), (int)N, (int)K, mult.data(), b >= 0 ? (const int32_t*)T(b).host.data() : nullptr, xzp, *prep);
                    const int aw = pl->add_aux(prep->w_blk.data(), prep->w_blk.size()), am = pl->add_aux(prep->mult.data(), prep->mult.size() * 4);
                    const int ab = pl->add_aux(prep->bias.data(), prep->bias.size() * 4);
                    const int sa = pl->shared_im2col_scratch(qgemm_a_bytes(M, *prep));
                    prep->w_blk.clear(); prep->w_blk.shrink_to_fit();
                    push("QLinearMatMul(tc)", [=]() {
                        return run_qconv_tc(ctx, g, pl->ptr(x), xd == ZANT_U8, xzp, *prep, (const int8_t*)pl->aux(aw), (const float*)pl->aux(am),
                                            (const int32_t*)pl->aux(ab), (uint8_t*)pl->scratch(sa), pl->ptr(y), yd == ZANT_U8, rq);
                    });
                    return ZANT_OK;
                }
            }
            const int am = pl->add_aux(mult.data(), mult.size() * 4), az = pl->add_aux(bz.data(), bz.size() * 4);
            push("QLinearMatMul", [=]() {
                QMatArgs q{};
                q.a = pl->ptr(x); q.b = pl->p<int8_t>(w); q.y = pl->ptr(y);
                q.mult = (const float*)pl->aux(am); q.b_zp = (const int32_t*)pl->aux(az); q.bias = pl->p<int32_t>(b);
                q.a_zp = xzp; q.rq = rq; q.M = (int)M; q.N = (int)N; q.K = (int)K; q.y_i32 = yd == ZANT_I32;
                return run_qmatmul_generic(ctx, q, xd, yd);
            });
            return ZANT_OK;
        }
        case ZANT_OP_QLINEAR_ADD: {
            ZB_TRY(need_inputs(n, 2, 2, "QLinearAdd"));
            const int x = n.in[0], w = n.in[1], y = n.out[0];
            const int32_t dt = T(x).dtype;
            if ((dt != ZANT_I8 && dt != ZANT_U8) || T(w).dtype != dt || T(y).dtype != dt) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearAdd dtypes");
            const size_t cnt = numel(T(x).shape.data(), T(x).shape.size());
            if (cnt != numel(T(w).shape.data(), T(w).shape.size()) || cnt != numel(T(y).shape.data(), T(y).shape.size()))
                return fail(ZANT_E_INPUT_TENSOR_DIFFERENT_SIZE, "QLinearAdd sizes differ");
            const zant_node_attrs aa = a;
            push("QLinearAdd", [=]() { return run_qadd(ctx, dt, pl->ptr(x), aa.x_scale, aa.x_zp, pl->ptr(w), aa.b_scale, aa.b_zp, aa.y_scale, aa.y_zp, aa.activation, pl->ptr(y), cnt); });
            return ZANT_OK;
        }
        case ZANT_OP_QLINEAR_GLOBAL_AVGPOOL: {
            ZB_TRY(need_inputs(n, 1, 1, "QLinearGlobalAveragePool"));
            const int x = n.in[0], y = n.out[0];
            const int32_t dt = T(x).dtype;
            if ((dt != ZANT_I8 && dt != ZANT_U8) || T(y).dtype != dt) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "QLinearGlobalAveragePool dtypes");
            if (T(x).shape.size() != 4) return fail(ZANT_E_INVALID_DIMENSIONS, "QLinearGlobalAveragePool needs a 4-D input");
            const size_t planes = T(x).shape[0] * T(x).shape[1], hw = T(x).shape[2] * T(x).shape[3];
            if (numel(T(y).shape.data(), T(y).shape.size()) != planes || hw == 0) return fail(ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE, "QLinearGlobalAveragePool output size");
            const zant_node_attrs aa = a;
            push("QLinearGlobalAveragePool", [=]() { return run_qgap(ctx, dt, pl->ptr(x), pl->ptr(y), planes, (int)hw, aa.x_scale, aa.x_zp, aa.y_scale, aa.y_zp); });
            return ZANT_OK;
        }
        case ZANT_OP_LUT_Q8: {
            ZB_TRY(need_inputs(n, 2, 2, "LutQ8"));
            const int x = n.in[0], l = n.in[1], y = n.out[0];
            if (T(l).bytes != 256) return fail(ZANT_E_INPUT_TENSORS_WRONG_SHAPE, "table must hold 256 bytes");
            const size_t cnt = T(x).bytes;
            if (dtype_size(T(x).dtype) != 1 || T(y).bytes != cnt) return fail(ZANT_E_INPUT_ARRAY_WRONG_TYPE, "LutQ8 works on 8-bit tensors of equal size");
            push("LutQ8", [=]() { return run_lut(ctx, pl->ptr(x), pl->ptr(y), cnt, pl->p<uint8_t>(l)); });
            return ZANT_OK;
        }
        default:
            return fail(ZANT_E_UNSUPPORTED, "operator %d is not supported", n.op);
    }
}

// --------------------------------------------------------------------------------------------
// Fusion.  `try_fuse` looks for a known chain starting at `node_index` and, if every shape,
// attribute and data-flow condition holds, emits fused steps and reports how many nodes they
// cover (0 = nothing matched; the caller builds the node on its own).
//
// Chain recognised today (the reference's example CNN in QLinear form):
//   QuantizeLinear(u8) -> QLinearConv(1->32,3x3) -> Relu -> MaxPool 2x2/2
//                      -> QLinearConv(32->64,3x3) -> Relu -> MaxPool 2x2/2 -> Reshape
//                      -> QLinearMatMul -> Relu -> QLinearMatMul -> DequantizeLinear
// on [N,1,28,28] inputs.  Intermediate tensors of a fused chain are not materialised in their
// graph layout: they live in private scratch buffers (C16-planar / GEMM-ordered).
// --------------------------------------------------------------------------------------------
namespace {

struct ChainCtx {
    zant_plan* pl;
    std::vector<int> consumers;   // per tensor: number of nodes reading it
};

bool only_feeds_next(const ChainCtx& c, int tensor) {
    return c.consumers[tensor] == 1 && tensor != c.pl->output && !c.pl->t[tensor].is_const;
}

bool shape_is(const PlanTensor& t, std::initializer_list<size_t> s) { return t.shape == std::vector<size_t>(s); }

bool plain_conv3x3(const zant_node_attrs& a) {
    auto one = [](const size_t* v, size_t n) { for (size_t i = 0; i < n; ++i) if (v[i] != 1) return false; return true; };
    bool nopad = true;
    for (size_t i = 0; i < a.n_pads; ++i) nopad = nopad && a.pads[i] == 0;
    return one(a.strides, a.n_strides) && one(a.dilations, a.n_dilations) && nopad && (a.group == 0 || a.group == 1) &&
           (a.auto_pad < 0 || a.auto_pad == ZANT_PAD_NOTSET || a.auto_pad == ZANT_PAD_VALID);
}

bool pool2x2(const zant_node_attrs& a) {
    bool nopad = true;
    for (size_t i = 0; i < a.n_pads; ++i) nopad = nopad && a.pads[i] == 0;
    const bool d1 = a.n_dilations == 0 || (a.dilations[0] == 1 && a.dilations[1] == 1);
    return a.kernel_shape[0] == 2 && a.kernel_shape[1] == 2 && a.n_strides == 2 && a.strides[0] == 2 && a.strides[1] == 2 && nopad && d1 &&
           (a.auto_pad < 0 || a.auto_pad == ZANT_PAD_NOTSET || a.auto_pad == ZANT_PAD_VALID);
}

// A quantized Relu node that keeps scale and zero point is max(q, zp): foldable into the producer.
bool identity_scale_relu(const PlanNode& n) {
    return n.op == ZANT_OP_RELU && n.a.x_scale == n.a.y_scale && n.a.x_zp == n.a.y_zp;
}

bool all_zero_i32(const PlanTensor& t) {
    const int32_t* v = (const int32_t*)t.host.data();
    for (size_t i = 0; i < t.bytes / 4; ++i) if (v[i] != 0) return false;
    return true;
}

bool positive_finite(const std::vector<float>& m) {
    for (float v : m) if (!(v > 0.0f) || !std::isfinite(v)) return false;
    return true;
}

}  // namespace

static int32_t try_fuse(zant_plan* pl, size_t i0, size_t& consumed) {
    consumed = 0;
    ZB_TRY(try_fuse_small_cnn(pl, i0, consumed));
    if (consumed) return ZANT_OK;
    ZB_TRY(try_fuse_qconv_group(pl, i0, consumed));
    if (consumed) return ZANT_OK;
    return try_fuse_fconv_group(pl, i0, consumed);
}

// Float Conv -> Relu | LeakyRelu on the tensor-core path (context in TF32 mode): the activation runs in the GEMM's
// epilogue.  The exact FP32 path is left node by node: it mirrors the reference's call sequence.
static int32_t try_fuse_fconv_group(zant_plan* pl, size_t i0, size_t& consumed) {
    consumed = 0;
    if (!pl->ctx->tf32 || i0 + 1 >= pl->nodes.size()) return ZANT_OK;
    const PlanNode& conv = pl->nodes[i0];
    const PlanNode& act = pl->nodes[i0 + 1];
    if (conv.op != ZANT_OP_CONV || conv.out.size() != 1) return ZANT_OK;
    if ((act.op != ZANT_OP_RELU && act.op != ZANT_OP_LEAKY_RELU) || act.in.size() != 1 || act.out.size() != 1 || act.in[0] != conv.out[0]) return ZANT_OK;
    if (pl->t[act.out[0]].dtype != ZANT_F32 || pl->t[act.out[0]].bytes != pl->t[conv.out[0]].bytes) return ZANT_OK;
    ChainCtx c{pl, std::vector<int>(pl->t.size(), 0)};
    for (const PlanNode& n : pl->nodes) for (int id : n.in) if (id >= 0) c.consumers[id]++;
    if (!only_feeds_next(c, conv.out[0])) return ZANT_OK;
    pl->pending_fact = act.op == ZANT_OP_RELU ? FACT_RELU : FACT_LEAKY;
    pl->pending_slope = act.a.alpha;
    pl->pending_y = act.out[0];
    pl->pending_used = false;
    const size_t first_step = pl->steps.size();
    const int32_t st = build_node_impl(pl, i0, 1);
    const bool used = pl->pending_used;
    pl->pending_fact = FACT_NONE; pl->pending_slope = 0.0f; pl->pending_y = -1; pl->pending_used = false;
    if (st != ZANT_OK) return st;
    if (used) { pl->t[conv.out[0]].elided = true; consumed = 2; }
    else consumed = 1;
    record_step_cost(pl, first_step, i0, consumed);
    return ZANT_OK;
}

// --------------------------------------------------------------------------------------------
// Generic epilogue fusion: QLinearConv -> [Relu | LeakyRelu | Clip] -> [MaxPool 2x2 / stride 2].
// The generator emits one call per node (src/codeGen/predict.zig:73-92, src/codeGen/math_handler.zig:45-105), so
// between a convolution and the pool behind it two full-size int8 tensors are written and read back.  Here the
// activation becomes part of the producer's epilogue (an activation flag when it keeps scale and zero point, else
// a 256-entry table applied to the finished code), and the pool is applied in the epilogue of the implicit-GEMM
// kernel where its tiling allows; the tensors in between are never materialised.  Every step is the composition of
// the exact per-node functions on the same integer codes, so results stay bit-identical to the node-by-node plan.
// Conditions: each interior tensor has exactly one consumer and is not the graph output; the pool has a 2x2
// window, stride 2, no padding, no dilation (MaxPool rule: src/Core/Tensor/TensorMath/op_pooling.zig:570-659).
// --------------------------------------------------------------------------------------------
static int32_t try_fuse_qconv_group(zant_plan* pl, size_t i0, size_t& consumed) {
    consumed = 0;
    const PlanNode& conv = pl->nodes[i0];
    if (conv.op != ZANT_OP_QLINEAR_CONV || conv.out.size() != 1 || conv.in.size() < 3) return ZANT_OK;
    ChainCtx c{pl, std::vector<int>(pl->t.size(), 0)};
    for (const PlanNode& n : pl->nodes) for (int id : n.in) if (id >= 0) c.consumers[id]++;
    auto T = [&](int id) -> const PlanTensor& { return pl->t[id]; };
    auto q8 = [&](int id) { return T(id).dtype == ZANT_I8 || T(id).dtype == ZANT_U8; };
    QConvFusion fz;
    size_t j = i0 + 1;
    int cur = conv.out[0];
    if (!q8(cur)) return ZANT_OK;
    std::vector<int> interior;
    // activation behind the convolution
    if (j < pl->nodes.size() && only_feeds_next(c, cur)) {
        const PlanNode& act = pl->nodes[j];
        const bool is_act = act.op == ZANT_OP_RELU || act.op == ZANT_OP_LEAKY_RELU || act.op == ZANT_OP_CLIP;
        if (is_act && act.in.size() == 1 && act.out.size() == 1 && act.in[0] == cur && T(act.out[0]).dtype == T(cur).dtype &&
            T(act.out[0]).bytes == T(cur).bytes && act.a.x_scale == conv.a.y_scale && act.a.x_zp == conv.a.y_zp) {
            if (identity_scale_relu(act)) {
                fz.activation = conv.a.activation == ZANT_QACT_NONE ? ZANT_QACT_RELU : conv.a.activation;
            } else {
                uint8_t lut[256];
                activation_lut(act, T(cur).dtype, lut);
                fz.lut_aux = pl->add_aux(lut, 256);
            }
            interior.push_back(cur);
            cur = act.out[0];
            ++j;
        }
    }
    // pool behind that
    bool want_pool = false;
    if (!conv.a.channels_last && j < pl->nodes.size() && only_feeds_next(c, cur)) {
        const PlanNode& pool = pl->nodes[j];
        if (pool.op == ZANT_OP_MAXPOOL && pool.in.size() == 1 && pool.out.size() == 1 && pool.in[0] == cur && pool2x2(pool.a) &&
            T(pool.out[0]).dtype == T(cur).dtype && T(cur).shape.size() == 4 && T(pool.out[0]).shape.size() == 4) {
            const auto& si = T(cur).shape; const auto& so = T(pool.out[0]).shape;
            if (so[0] == si[0] && so[1] == si[1] && so[2] == si[2] / 2 && so[3] == si[3] / 2 && so[2] > 0 && so[3] > 0) {
                want_pool = true;
                fz.y_pool = pool.out[0];
            }
        }
    }
    if (interior.empty() && !want_pool) return ZANT_OK;        // nothing behind the node: the plain path builds it
    fz.y_act = cur;
    const size_t first_step = pl->steps.size();
    ZB_TRY(build_qconv(pl, conv, fz));
    if (fz.pool_done) { interior.push_back(cur); ++j; }
    if (interior.empty()) {
        // the pool was asked for but the chosen kernel cannot take it: nothing was fused after all
        record_step_cost(pl, first_step, i0, 1);
        consumed = 1;
        return ZANT_OK;
    }
    for (int id : interior) pl->t[id].elided = true;
    consumed = j - i0;
    record_step_cost(pl, first_step, i0, consumed);
    return ZANT_OK;
}

static int32_t try_fuse_small_cnn(zant_plan* pl, size_t i0, size_t& consumed) {
    consumed = 0;
    if (i0 + 12 > pl->nodes.size()) return ZANT_OK;
    const int kOps[12] = {ZANT_OP_QUANTIZE_LINEAR, ZANT_OP_QLINEAR_CONV, ZANT_OP_RELU, ZANT_OP_MAXPOOL, ZANT_OP_QLINEAR_CONV, ZANT_OP_RELU,
                          ZANT_OP_MAXPOOL, ZANT_OP_RESHAPE, ZANT_OP_QLINEAR_MATMUL, ZANT_OP_RELU, ZANT_OP_QLINEAR_MATMUL, ZANT_OP_DEQUANTIZE_LINEAR};
    for (int k = 0; k < 12; ++k) if (pl->nodes[i0 + k].op != kOps[k]) return ZANT_OK;
    ChainCtx c{pl, std::vector<int>(pl->t.size(), 0)};
    for (const PlanNode& n : pl->nodes) for (int id : n.in) if (id >= 0) c.consumers[id]++;
    const PlanNode* N = &pl->nodes[i0];
    auto T = [&](int id) -> const PlanTensor& { return pl->t[id]; };
    // data flow: each node's first input is the previous node's only output, used nowhere else
    for (int k = 1; k < 12; ++k) {
        if (N[k].in.empty() || N[k - 1].out.size() != 1 || N[k].in[0] != N[k - 1].out[0]) return ZANT_OK;
        if (!only_feeds_next(c, N[k - 1].out[0])) return ZANT_OK;
    }
    const int x = N[0].in[0], y = N[11].out[0];
    if (T(x).dtype != ZANT_F32 || T(x).shape.size() != 4) return ZANT_OK;
    const size_t B = T(x).shape[0];
    if (B == 0 || B > 0x3fffffffULL) return ZANT_OK;
    if (!shape_is(T(x), {B, 1, 28, 28}) || T(N[0].out[0]).dtype != ZANT_U8) return ZANT_OK;
    // conv1
    const PlanNode& c1 = N[1];
    if (c1.in.size() < 3 || !plain_conv3x3(c1.a) || !shape_is(T(c1.in[1]), {32, 1, 3, 3}) || !shape_is(T(c1.out[0]), {B, 32, 26, 26})) return ZANT_OK;
    if (T(c1.out[0]).dtype != ZANT_I8 || c1.a.activation == ZANT_QACT_RELU6 || c1.a.y_zp != 0) return ZANT_OK;
    if (c1.a.x_scale != N[0].a.y_scale || c1.a.x_zp != N[0].a.y_zp) return ZANT_OK;
    if (opt_in(c1, 3) >= 0 && !all_zero_i32(T(c1.in[3]))) return ZANT_OK;
    if (!identity_scale_relu(N[2]) || N[2].a.x_scale != c1.a.y_scale || N[2].a.x_zp != c1.a.y_zp) return ZANT_OK;
    if (!pool2x2(N[3].a) || !shape_is(T(N[3].out[0]), {B, 32, 13, 13})) return ZANT_OK;
    // conv2
    const PlanNode& c2 = N[4];
    if (c2.in.size() < 3 || !plain_conv3x3(c2.a) || !shape_is(T(c2.in[1]), {64, 32, 3, 3}) || !shape_is(T(c2.out[0]), {B, 64, 11, 11})) return ZANT_OK;
    if (T(c2.out[0]).dtype != ZANT_I8 || c2.a.activation == ZANT_QACT_RELU6 || c2.a.y_zp != 0) return ZANT_OK;
    if (c2.a.x_scale != c1.a.y_scale || c2.a.x_zp != c1.a.y_zp) return ZANT_OK;
    if (opt_in(c2, 3) >= 0 && !all_zero_i32(T(c2.in[3]))) return ZANT_OK;
    if (!identity_scale_relu(N[5]) || N[5].a.x_scale != c2.a.y_scale || N[5].a.x_zp != c2.a.y_zp) return ZANT_OK;
    if (!pool2x2(N[6].a) || !shape_is(T(N[6].out[0]), {B, 64, 5, 5})) return ZANT_OK;
    if (!shape_is(T(N[7].out[0]), {B, 1600})) return ZANT_OK;
    // fc1, fc2
    const PlanNode& f1 = N[8];
    const PlanNode& f2 = N[10];
    if (f1.in.size() < 3 || f2.in.size() < 3) return ZANT_OK;
    if (!shape_is(T(f1.in[1]), {1600, 512}) || !shape_is(T(f1.out[0]), {B, 512}) || T(f1.out[0]).dtype != ZANT_I8) return ZANT_OK;
    if (f1.a.x_scale != c2.a.y_scale || f1.a.x_zp != c2.a.y_zp || f1.a.activation == ZANT_QACT_RELU6 || f1.a.y_zp != 0) return ZANT_OK;
    if (opt_in(f1, 3) >= 0 && !all_zero_i32(T(f1.in[3]))) return ZANT_OK;
    if (!identity_scale_relu(N[9]) || N[9].a.x_scale != f1.a.y_scale || N[9].a.x_zp != f1.a.y_zp) return ZANT_OK;
    if (T(f2.in[1]).shape.size() != 2 || T(f2.in[1]).shape[0] != 512 || T(f2.out[0]).dtype != ZANT_I8) return ZANT_OK;
    const size_t NCLS = T(f2.in[1]).shape[1];
    if (NCLS == 0 || NCLS > 64 || !shape_is(T(f2.out[0]), {B, NCLS}) || !shape_is(T(y), {B, NCLS})) return ZANT_OK;
    if (f2.a.x_scale != f1.a.y_scale || f2.a.x_zp != f1.a.y_zp || f2.a.activation != ZANT_QACT_NONE) return ZANT_OK;
    if (opt_in(f2, 3) >= 0 && !all_zero_i32(T(f2.in[3]))) return ZANT_OK;
    if (N[11].a.x_scale != f2.a.y_scale || N[11].a.x_zp != f2.a.y_zp || T(y).dtype != ZANT_F32) return ZANT_OK;
    for (const PlanNode* q : {&c1, &c2, &f1, &f2})
        for (size_t k = 1; k < q->in.size(); ++k)
            if (q->in[k] >= 0 && !T(q->in[k]).is_const) return ZANT_OK;

    zant_ctx* ctx = pl->ctx;
    auto push = [&](const char* name, std::function<int32_t()> fn) { pl->steps.push_back(std::move(fn)); pl->step_names.push_back(name); };
    auto scales_of = [&](const PlanNode& q, size_t M, std::vector<float>& mult) {
        const PlanTensor& ws = T(q.in[2]);
        const size_t nws = ws.bytes / 4;
        if (ws.dtype != ZANT_F32 || (nws != 1 && nws != M)) return false;
        requant_multipliers(q.a.x_scale, (const float*)ws.host.data(), nws, q.a.y_scale, M, mult);
        return positive_finite(mult);
    };
    auto bias_of = [&](const PlanNode& q, size_t M, std::vector<int32_t>& bias) {
        bias.assign(M, 0);
        const int b = opt_in(q, 4);
        if (b < 0) return true;
        if (T(b).dtype != ZANT_I32 || T(b).bytes != M * 4) return false;
        std::memcpy(bias.data(), T(b).host.data(), M * 4);
        return true;
    };

    // ---- stage 1 parameters (weights travel as kernel parameters)
    std::vector<float> m1; std::vector<int32_t> b1;
    if (!scales_of(c1, 32, m1) || !bias_of(c1, 32, b1)) return ZANT_OK;
    Conv1Args a1{};
    {
        const int8_t* w = (const int8_t*)T(c1.in[1]).host.data();
        for (int m = 0; m < 32; ++m) {
            int sum = 0;
            for (int kh = 0; kh < 3; ++kh) {
                const uint32_t w0 = (uint8_t)w[m * 9 + kh * 3 + 0], w1 = (uint8_t)w[m * 9 + kh * 3 + 1], w2 = (uint8_t)w[m * 9 + kh * 3 + 2];
                a1.wpack[m][kh][0] = w0 | (w1 << 8) | (w2 << 16);
                a1.wpack[m][kh][1] = (w0 << 8) | (w1 << 16) | (w2 << 24);
                sum += w[m * 9 + kh * 3] + w[m * 9 + kh * 3 + 1] + w[m * 9 + kh * 3 + 2];
            }
            a1.mult[m] = m1[m];
            a1.bias[m] = b1[m] - c1.a.x_zp * sum;
        }
        a1.n_images = (int)B; a1.x_scale = N[0].a.y_scale; a1.x_zp = N[0].a.y_zp;
        a1.y_scale = c1.a.y_scale; a1.y_zp = c1.a.y_zp; a1.act = ZANT_QACT_RELU;
    }
    // ---- stage 2 parameters
    std::vector<float> m2; std::vector<int32_t> b2;
    if (!scales_of(c2, 64, m2) || !bias_of(c2, 64, b2)) return ZANT_OK;
    std::vector<int8_t> w2arr(TcConvParityCfg::W_ALL_BYTES);      // nine taps, then the paired blocks
    {
        const int8_t* w = (const int8_t*)T(c2.in[1]).host.data();   // [64][32][3][3]
        for (int m = 0; m < 64; ++m) {
            int sum = 0;
            for (int ch = 0; ch < 32; ++ch)
                for (int tap = 0; tap < 9; ++tap) {
                    const int8_t v = w[(m * 32 + ch) * 9 + tap];
                    w2arr[((tap * 2 + ch / 16) * 64 + m) * 16 + ch % 16] = v;
                    sum += v;
                }
            b2[m] -= c2.a.x_zp * sum;
        }
        // paired blocks [kh][j][chunk][128 rows][16]: rows 0-63 tap (kh, j + 1), rows 64-127 tap (kh, j)
        for (int kh = 0; kh < 3; ++kh)
            for (int j = 0; j < 2; ++j)
                for (int chunk = 0; chunk < 2; ++chunk)
                    for (int r = 0; r < 128; ++r) {
                        const int tap = kh * 3 + (r < 64 ? j + 1 : j), m = r & 63;
                        std::memcpy(&w2arr[TcConvParityCfg::W_BYTES + (size_t)(((kh * 2 + j) * 2 + chunk) * 128 + r) * 16],
                                    &w2arr[(size_t)((tap * 2 + chunk) * 64 + m) * 16], 16);
                    }
    }
    // ---- fc1: rows re-ordered from the graph's (c,h,w) flatten order to the (h,w,c) order stage 2 writes
    std::vector<float> m3; std::vector<int32_t> b3;
    if (!scales_of(f1, 512, m3) || !bias_of(f1, 512, b3)) return ZANT_OK;
    constexpr int FC_NT = 256, FC_KC = 4, FC_STAGES = 8;
    std::vector<int8_t> w3blk(1600 * 512);      // [512/NT][100 chunks][NT][16], K in (h,w,c) order
    {
        const int8_t* w = (const int8_t*)T(f1.in[1]).host.data();   // [1600][512], row = c*25 + h*5 + w
        std::vector<int> colsum(512, 0);
        for (int ch = 0; ch < 64; ++ch)
            for (int hw = 0; hw < 25; ++hw) {
                const int k = hw * 64 + ch;                         // position in the order stage 2 writes
                const int8_t* src = &w[(size_t)(ch * 25 + hw) * 512];
                for (int n = 0; n < 512; ++n) {
                    w3blk[(((size_t)(n / FC_NT) * 100 + k / 16) * FC_NT + n % FC_NT) * 16 + k % 16] = src[n];
                    colsum[n] += src[n];
                }
            }
        for (int n = 0; n < 512; ++n) b3[n] -= f1.a.x_zp * colsum[n];
    }
    std::vector<float> m4; std::vector<int32_t> b4;
    if (!scales_of(f2, NCLS, m4) || !bias_of(f2, NCLS, b4)) return ZANT_OK;
    if (NCLS > 16) return ZANT_OK;
    {
        const int8_t* w = (const int8_t*)T(f2.in[1]).host.data();   // [512][NCLS]
        for (size_t n = 0; n < NCLS; ++n) {
            int sum = 0;
            for (int k = 0; k < 512; ++k) sum += w[(size_t)k * NCLS + n];
            b4[n] -= f2.a.x_zp * sum;
        }
    }

    // stage 1 -> stage 2 hand-over: parity planes (TcConvParityCfg), every tile of stage 2 copies 136 rows of each plane
    if (B > (1u << 20)) return ZANT_OK;                     // 32-bit plane offsets in stage 1
    const long long c2_tiles = ((long long)B * 36 + 127) / 128;
    const long long plane_bytes = (TcConvParityCfg::plane_rows(c2_tiles) * 16 + 255) / 256 * 256;
    const int s_pool1 = pl->add_scratch((size_t)(8 * plane_bytes));
    const size_t Bpad = (B + 127) / 128 * 128;
    const int s_pool2 = pl->add_scratch(Bpad * 1600);
    const int s_fc1 = pl->add_scratch(B * 512);
    const int a_w2 = pl->add_aux(w2arr.data(), w2arr.size());
    const int a_w3 = pl->add_aux(w3blk.data(), w3blk.size());
    const int a_m3 = pl->add_aux(m3.data(), m3.size() * 4), a_b3 = pl->add_aux(b3.data(), b3.size() * 4);
    const int a_m4 = pl->add_aux(m4.data(), m4.size() * 4), a_b4 = pl->add_aux(b4.data(), b4.size() * 4);
    const int w4 = f2.in[1];

    // B-fragment words, bias and multipliers in the per-lane order of the warp-level MMA
    std::vector<uint32_t> wfrag(4 * 4 * 32);
    std::vector<int32_t> biasfrag(4 * 32 * 2);
    std::vector<float> multfrag(4 * 32 * 2);
    {
        const int8_t* w = (const int8_t*)T(c1.in[1]).host.data();   // [32][1][3][3]
        for (int lane = 0; lane < 32; ++lane) {
            const int g = lane >> 2, t = lane & 3;
            for (int j = 0; j < 4; ++j) {
                const int ch = 8 * (g / 2) + 2 * j + (g % 2);        // column g of channel group j
                for (int m = 0; m < 4; ++m) {
                    const int dy = m >> 1, dx = m & 1, kh = t - dy;
                    uint32_t word = 0;
                    for (int sx = 0; sx < 4; ++sx) {
                        const int kw = sx - dx;
                        if (kh >= 0 && kh < 3 && kw >= 0 && kw < 3) word |= (uint32_t)(uint8_t)w[ch * 9 + kh * 3 + kw] << (8 * sx);
                    }
                    wfrag[(m * 4 + j) * 32 + lane] = word;
                }
                for (int b = 0; b < 2; ++b) {
                    const int cc = 8 * t + 2 * j + b;                // the lane's accumulator columns 2t, 2t+1
                    biasfrag[(j * 32 + lane) * 2 + b] = a1.bias[cc];
                    multfrag[(j * 32 + lane) * 2 + b] = a1.mult[cc];
                }
            }
        }
    }
    const int a_wf = pl->add_aux(wfrag.data(), wfrag.size() * 4);
    const int a_bf = pl->add_aux(biasfrag.data(), biasfrag.size() * 4);
    const int a_mf = pl->add_aux(multfrag.data(), multfrag.size() * 4);
    push("Fused[QuantizeLinear+QLinearConv+Relu+MaxPool] mma", [=]() {
        Conv1MmaArgs k{};
        k.x = pl->p<float>(x); k.y = (int8_t*)pl->scratch(s_pool1); k.n_images = (int)B;
        k.x_scale = a1.x_scale; k.x_zp = a1.x_zp;
        k.wfrag = (const uint32_t*)pl->aux(a_wf); k.biasfrag = (const int32_t*)pl->aux(a_bf); k.multfrag = (const float*)pl->aux(a_mf); k.status = ctx->status_word; k.plane_bytes = plane_bytes;
        const int blocks = std::min<int>((int)((B + C1M_G - 1) / C1M_G), ctx->sm_count * 8);
        conv1_mma_relu_pool_kernel<<<blocks, C1M_THREADS, 0, ctx->stream>>>(k);
        return check_launch(ctx, "conv1_mma_relu_pool_kernel");
    });
    push("Fused[QLinearConv+Relu+MaxPool] tcgen05", [=]() {
        using Cfg = TcConvParityCfg;
        ZB_SMEM_ATTR(ctx, (tc_conv3x3_pool_parity_kernel), Cfg::SMEM_BYTES);
        TcConvParityArgs k{};
        k.x = (const int8_t*)pl->scratch(s_pool1); k.plane_bytes = plane_bytes; k.w = (const int8_t*)pl->aux(a_w2);
        for (int m = 0; m < 64; ++m) { k.mult[m] = m2[m]; k.bias[m] = b2[m]; }
        k.y = (int8_t*)pl->scratch(s_pool2); k.n_images = (int)B; k.n_tiles = (int)c2_tiles; k.status = ctx->status_word;
        const int blocks = std::min<int>((int)c2_tiles, ctx->sm_count);
        tc_conv3x3_pool_parity_kernel<<<blocks, Cfg::THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(k);
        return check_launch(ctx, "tc_conv3x3_pool_parity_kernel");
    });
    const zant_node_attrs f1a = f1.a, f2a = f2.a, dqa = N[11].a;
    push("Fused[Reshape+QLinearMatMul+Relu] tcgen05", [=]() {
        using Cfg = TcGemmCfg<FC_NT, FC_KC, FC_STAGES>;
        ZB_SMEM_ATTR(ctx, (tc_gemm_i8_kernel<FC_NT, FC_KC, FC_STAGES>), Cfg::SMEM_BYTES);
        TcGemmArgs k{};
        k.a = (const int8_t*)pl->scratch(s_pool2); k.w = (const int8_t*)pl->aux(a_w3);
        k.mult = (const float*)pl->aux(a_m3); k.bias = (const int32_t*)pl->aux(a_b3);
        k.y = (int8_t*)pl->scratch(s_fc1); k.M = (int)B; k.N = 512; k.K16 = 100;
        k.y_scale = f1a.y_scale; k.y_zp = f1a.y_zp; k.act = ZANT_QACT_RELU; k.status = ctx->status_word;
        const int tiles = (int)((B + 127) / 128) * (512 / FC_NT);
        const int blocks = std::min(tiles, ctx->sm_count);
        tc_gemm_i8_kernel<FC_NT, FC_KC, FC_STAGES><<<blocks, Cfg::THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(k);
        return check_launch(ctx, "tc_gemm_i8_kernel");
    });
    push("Fused[QLinearMatMul+DequantizeLinear]", [=]() {
        FcOutArgs k{};
        k.a = (const int8_t*)pl->scratch(s_fc1); k.w = pl->p<int8_t>(w4);
        k.mult = (const float*)pl->aux(a_m4); k.bias = (const int32_t*)pl->aux(a_b4);
        k.y = pl->p<float>(y); k.M = (int)B; k.K = 512; k.NCLS = (int)NCLS;
        k.y_scale = f2a.y_scale; k.y_zp = f2a.y_zp; k.dq_scale = dqa.x_scale; k.dq_zp = dqa.x_zp;
        // one or two column blocks of 8 classes
        auto launch = [&](auto nc) -> int32_t {
            constexpr int NC = decltype(nc)::value;
            constexpr int smem = fcout_smem_bytes<NC, 512>();
            ZB_SMEM_ATTR(ctx, (fc_out_dequant_kernel<NC, 512>), smem);
            const int blocks = std::min<int>((int)((B + 127) / 128), ctx->sm_count * 3);
            fc_out_dequant_kernel<NC, 512><<<blocks, FCOUT_THREADS, smem, ctx->stream>>>(k);
            return check_launch(ctx, "fc_out_dequant_kernel");
        };
        return NCLS <= 8 ? launch(std::integral_constant<int, 8>{}) : launch(std::integral_constant<int, 16>{});
    });
    for (int k = 0; k < 11; ++k) pl->t[N[k].out[0]].elided = true;   // interior tensors live only inside the fused kernels
    consumed = 12;
    {
        // algorithmic work of the four fused steps: tensors that cross a kernel boundary once at their storage type,
        // weights included; of the 13 x 13 pooled pixels of stage 1 only the 12 x 12 that stage 2's pool reads exist
        const double Bd = (double)B, nc = (double)NCLS;
        const double macs[4] = {Bd * 194688.0, Bd * 2230272.0, Bd * 819200.0, Bd * 512.0 * nc};
        const double bytes[4] = {Bd * (784.0 * 4 + 144.0 * 32) + 288.0, Bd * (144.0 * 32 + 1600.0) + 64.0 * 288, Bd * (1600.0 + 512.0) + 1600.0 * 512,
                                 Bd * (512.0 + 4.0 * nc) + 512.0 * nc};
        pl->step_macs.resize(pl->steps.size(), 0.0); pl->step_bytes.resize(pl->steps.size(), 0.0);
        for (int k = 0; k < 4; ++k) { pl->step_macs[pl->steps.size() - 4 + k] = macs[k]; pl->step_bytes[pl->steps.size() - 4 + k] = bytes[k]; }
    }
    return ZANT_OK;
}
