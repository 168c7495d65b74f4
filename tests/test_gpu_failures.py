"""Failure paths on a healthy GPU: every test here makes the failure on the host, or lets a bounded
device-side wait run out; nothing faults, traps or hangs the device.  Error names follow the
reference's error sets (src/Utils/errorHandler.zig:36-84); generated code reacts to any of them
with `catch return` (src/codeGen/math_handler.zig:107), so what matters is that the call fails
cleanly and the context keeps working."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
I8, U8 = 1, 2


def _small_conv(ctx, oracle):
    rng = np.random.default_rng(5)
    x = rng.integers(-128, 128, (2, 16, 8, 8), dtype=np.int8)
    w = rng.integers(-127, 128, (16, 16, 3, 3), dtype=np.int8)
    kw = dict(stride=(1, 1), pads=(1, 1, 1, 1), dilations=(1, 1), group=1)
    got = ctx.qlinearconv(x, 0.02, 0, w, [0.02], None, 0.5, 0, **kw)
    want = oracle.qlinearconv(x, 0.02, 0, w, np.array([0.02], np.float32), None, 0.5, 0, **kw)
    assert np.array_equal(got, want)


def test_bounded_wait_times_out_and_context_survives(zb, oracle):
    """A wait that nothing satisfies gives up after its budget: the kernel frees its tensor memory and returns,
    the next synchronisation reports DeviceTimeout once, and the same context then computes correctly."""
    ctx = zb.Context(0)
    try:
        ctx.selftest_bounded_wait(budget_us=200)
        with pytest.raises(zb.ZantError) as e:
            ctx.synchronize()
        assert e.value.name == "DeviceTimeout"
        ctx.synchronize()                      # reported once, then cleared
        _small_conv(ctx, oracle)               # tensor-core path after the time-out: TMEM was released
        # a host-buffer call picks the time-out up itself (it waits for the stream anyway)
        ctx.selftest_bounded_wait(budget_us=50)
        with pytest.raises(zb.ZantError) as e:
            ctx.ReLU(np.ones(8, np.float32))
        assert e.value.name == "DeviceTimeout"
        assert np.array_equal(ctx.ReLU(np.array([-1.0, 2.0], np.float32)), np.array([0.0, 2.0], np.float32))
    finally:
        ctx.close()


def test_bad_device_index(zb):
    n = zb.device_count()
    for bad in (-1, n, n + 7):
        with pytest.raises(zb.ZantError) as e:
            zb.Context(bad)
        assert e.value.name == "InvalidInput"


def test_allocation_failure_is_mem_error(zb, oracle):
    """The allocator hook makes the next device allocation fail: context creation, host-buffer staging and
    plan finalisation each return MemError and leave everything usable."""
    from zant_b200 import models
    zb.debug_fail_alloc(1)
    with pytest.raises(zb.ZantError) as e:
        zb.Context(0)
    assert e.value.name == "MemError"
    ctx = zb.Context(0, arena_bytes=1 << 20)
    try:
        big = np.ones(1 << 20, np.float32)               # 8 MiB of staging: the arena has to grow
        zb.debug_fail_alloc(1)
        with pytest.raises(zb.ZantError) as e:
            ctx.ReLU(big)
        assert e.value.name == "MemError"
        assert np.array_equal(ctx.ReLU(big), big)        # the retry allocates for real
        g = models.small_cnn_int8(2)
        zb.debug_fail_alloc(1)
        with pytest.raises(zb.ZantError) as e:
            zb.Plan(ctx, g)
        assert e.value.name == "MemError"
        plan = zb.Plan(ctx, g)
        assert plan.run(models.small_cnn_input(2)).shape == (2, 10)
        plan.close()
        _small_conv(ctx, oracle)
    finally:
        zb.debug_fail_alloc(0)
        ctx.close()


def test_arena_limit(zb):
    ctx = zb.Context(0, arena_bytes=1 << 20)
    try:
        ctx.set_arena_limit(2 << 20)
        with pytest.raises(zb.ZantError) as e:
            ctx.ReLU(np.ones(1 << 20, np.float32))       # needs 8 MiB
        assert e.value.name == "ArenaExhausted"
        small = np.linspace(-1, 1, 1000, dtype=np.float32)
        assert np.array_equal(ctx.ReLU(small), np.maximum(small, 0))
        ctx.set_arena_limit(0)
        assert ctx.ReLU(np.ones(1 << 20, np.float32)).sum() == 1 << 20
    finally:
        ctx.close()


def test_bad_handles_and_unfinished_plans(zb, ctx):
    import ctypes as C
    L = zb.lib()
    assert L.zant_b200_plan_run(None, None, None) == -105                      # BadHandle
    h = C.c_void_p(None)
    assert L.zant_b200_plan_create(ctx._h, C.byref(h)) == 0
    buf = np.zeros(4, np.float32)
    assert L.zant_b200_plan_run(h, buf.ctypes.data_as(C.c_void_p), buf.ctypes.data_as(C.c_void_p)) == -105   # not finalized
    assert L.zant_b200_plan_finalize(h, C.c_int32(0), C.c_int32(0), C.c_int32(1)) == -55                     # no tensors: InvalidInput
    assert L.zant_b200_plan_destroy(h) == 0
    assert L.zant_b200_predict_sharded(None, None, None, C.c_size_t(1), None) == -105


def test_out_of_range_zero_points_are_refused(zb, ctx):
    x = np.zeros((1, 4, 4, 4), np.int8)
    w = np.zeros((4, 4, 1, 1), np.int8)
    for dt, zp in ((I8, 128), (I8, -129), (U8, -1), (U8, 256)):
        with pytest.raises(zb.ZantError) as e:
            ctx.qlinearconv(x.view(np.uint8) if dt == U8 else x, 0.1, zp, w, [0.1], None, 0.1, 0)
        assert e.value.name == "InvalidInput"
    with pytest.raises(zb.ZantError) as e:
        ctx.qlinearmatmul(np.zeros((2, 4), np.int8), 0.1, 300, np.zeros((4, 3), np.int8), [0.1], None, 0.1, 0)
    assert e.value.name == "InvalidInput"


def test_sharded_predict_reports_per_device_status(zb, oracle):
    """Two shards on one GPU (two contexts): results equal the single-plan run; a shard whose plan does not
    match its share of the batch is refused; and a device-side time-out in one shard comes back as that
    shard's status while the other shard's samples are still delivered."""
    import graph_oracle
    from zant_b200 import models
    batch = 10
    x = models.small_cnn_input(batch, 42)
    sp = zb.ShardedPredict(lambda n: models.small_cnn_int8(n), batch, devices=[0, 0])
    try:
        assert sp.world == 2
        y = sp.run(x)
        want = graph_oracle.run(oracle, models.small_cnn_int8(batch), x)
        assert np.array_equal(y, want[models.small_cnn_int8(batch).output])
        # one shard's context has a pending time-out: its status says so, the other shard is fine
        sp.contexts[1].selftest_bounded_wait(budget_us=50)
        y2, rc, status = sp.run(x, return_status=True)
        assert status[0] == 0 and status[1] == -106 and rc == -106
        assert np.array_equal(y2[:5], y[:5])
        y3, rc, status = sp.run(x, return_status=True)      # cleared: both fine again
        assert rc == 0 and status == [0, 0] and np.array_equal(y3, y)
        import ctypes as C
        rc = zb.lib().zant_b200_predict_sharded(sp._h, x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), C.c_size_t(batch + 2), None)
        assert rc == -3                                       # InputTensorDifferentSize: plans hold 5 + 5 samples
    finally:
        sp.close()
