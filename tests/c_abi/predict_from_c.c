/* A host written in C, as a compiled caller of the library would be: no Python, only include/zant_b200.h.
 *
 *   predict_from_c            with a GPU: runs a convolution from the reference's own unit test
 *                             (tests/Core/Tensor/TensorMath/test_op_convolution.zig:654-709: 5x5 ones,
 *                             3x3 ones filter -> nine everywhere) and a three-node plan
 *                             (Conv -> Relu -> MaxPool) on host buffers, and checks the numbers;
 *   without a GPU:            zant_b200_ctx_create must fail with CudaUnavailable, and the shape helpers
 *                             (host-only) must still work.
 * Exit code 0 = everything behaved as described, otherwise the number of the failed check. */
#include <stdio.h>
#include <string.h>

#include "zant_b200.h"

#define CHECK(n, cond) do { if (!(cond)) { fprintf(stderr, "check %d failed: %s (last error: %s)\n", n, #cond, zant_b200_last_error()); return n; } } while (0)

int main(void) {
    /* host-only helper: Slice output shape, reference test_lib_shape_math.zig:1050-1059 */
    size_t in_shape[3] = {5, 5, 5}, out_shape[3] = {0, 0, 0};
    int64_t starts[3] = {1, 1, 1}, ends[3] = {4, 4, 4}, steps[3] = {2, 2, 2};
    CHECK(1, zant_b200_slice_output_shape(in_shape, 3, starts, ends, 3, NULL, steps, out_shape) == ZANT_OK);
    CHECK(2, out_shape[0] == 2 && out_shape[1] == 2 && out_shape[2] == 2);

    zant_ctx* ctx = NULL;
    int32_t st = zant_b200_ctx_create(0, 0, &ctx);
    if (st != ZANT_OK) {
        /* no device: the library must say so and must not have produced a context */
        CHECK(3, st == ZANT_E_CUDA_UNAVAILABLE && ctx == NULL);
        CHECK(4, strcmp(zant_b200_status_name(st), "CudaUnavailable") == 0);
        printf("no GPU: %s, as expected\n", zant_b200_status_name(st));
        return 0;
    }

    /* single operator on host buffers */
    float x[25], w[9], y[9];
    for (int i = 0; i < 25; ++i) x[i] = 1.0f;
    for (int i = 0; i < 9; ++i) w[i] = 1.0f;
    size_t xs[4] = {1, 1, 5, 5}, ws[4] = {1, 1, 3, 3}, ys[4] = {1, 1, 3, 3}, stride[1] = {1}, pads[4] = {0, 0, 0, 0};
    CHECK(5, zant_b200_conv_f32(ctx, x, xs, 4, w, ws, 4, NULL, 0, y, ys, 4, stride, 1, pads, 4, NULL, 0, 0, NULL, 0) == ZANT_OK);
    for (int i = 0; i < 9; ++i) CHECK(6, y[i] == 9.0f);

    /* the same convolution as the first node of a plan: Conv -> Relu -> MaxPool 2x2 stride 1 */
    zant_plan* plan = NULL;
    CHECK(7, zant_b200_plan_create(ctx, &plan) == ZANT_OK);
    int32_t tx, tw, tc, tr, tp;
    size_t ps[4] = {1, 1, 2, 2};
    CHECK(8, zant_b200_plan_tensor(plan, ZANT_F32, xs, 4, NULL, &tx) == ZANT_OK);
    CHECK(9, zant_b200_plan_tensor(plan, ZANT_F32, ws, 4, w, &tw) == ZANT_OK);
    CHECK(10, zant_b200_plan_tensor(plan, ZANT_F32, ys, 4, NULL, &tc) == ZANT_OK);
    CHECK(11, zant_b200_plan_tensor(plan, ZANT_F32, ys, 4, NULL, &tr) == ZANT_OK);
    CHECK(12, zant_b200_plan_tensor(plan, ZANT_F32, ps, 4, NULL, &tp) == ZANT_OK);
    zant_node_attrs a;
    memset(&a, 0, sizeof a);
    a.strides[0] = 1; a.n_strides = 1; a.pads[0] = a.pads[1] = a.pads[2] = a.pads[3] = 0; a.n_pads = 4; a.auto_pad = -1;
    int32_t conv_in[3] = {tx, tw, -1};
    CHECK(13, zant_b200_plan_node(plan, ZANT_OP_CONV, conv_in, 3, &tc, 1, &a) == ZANT_OK);
    memset(&a, 0, sizeof a);
    a.auto_pad = -1;
    CHECK(14, zant_b200_plan_node(plan, ZANT_OP_RELU, &tc, 1, &tr, 1, &a) == ZANT_OK);
    memset(&a, 0, sizeof a);
    a.kernel_shape[0] = a.kernel_shape[1] = 2; a.strides[0] = a.strides[1] = 1; a.n_strides = 2;
    a.dilations[0] = a.dilations[1] = 1; a.n_dilations = 2; a.n_pads = 4; a.auto_pad = ZANT_PAD_NOTSET;
    CHECK(15, zant_b200_plan_node(plan, ZANT_OP_MAXPOOL, &tr, 1, &tp, 1, &a) == ZANT_OK);
    CHECK(16, zant_b200_plan_finalize(plan, tx, tp, 1) == ZANT_OK);
    float out[4] = {0, 0, 0, 0};
    x[12] = -100.0f;                                   /* centre pixel: every window sees it */
    CHECK(17, zant_b200_plan_run(plan, x, out) == ZANT_OK);
    for (int i = 0; i < 4; ++i) CHECK(18, out[i] == 0.0f);   /* 8 - 100 < 0 everywhere -> ReLU -> 0 */
    x[12] = 1.0f;
    CHECK(19, zant_b200_plan_use_graph(plan, 1) == ZANT_OK);
    CHECK(20, zant_b200_plan_run(plan, x, out) == ZANT_OK);
    for (int i = 0; i < 4; ++i) CHECK(21, out[i] == 9.0f);
    CHECK(22, zant_b200_plan_destroy(plan) == ZANT_OK);
    CHECK(23, zant_b200_ctx_destroy(ctx) == ZANT_OK);
    printf("C host: convolution, plan and graph replay agree with the reference's numbers\n");
    return 0;
}
