"""zant_b200_qlinearconv_noalloc: the QLinearConv entry point for callers that may not allocate.

A caller with a fixed memory budget (or one that mirrors Z-Ant's static-array-only generated code)
cannot create a Context, because a Context owns a cudaMalloc'd arena.  The no-allocation variant
keeps its per-channel constants in a fixed device array inside the library.  This test calls it
through the C ABI several times in a row with different layer shapes — each later call finds the
previous call's constants still in the shared array and must overwrite what it uses — and requires
bit-identical results to the regular entry point and to the CPU oracle.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
I8, U8 = 1, 2


def _case(rng, N, C, H, W, M, k, group, xdt, per_channel):
    x = rng.integers(0, 256, (N, C, H, W), dtype=np.uint8) if xdt == U8 else rng.integers(-128, 128, (N, C, H, W), dtype=np.int8)
    w = rng.integers(-127, 128, (M, C // group, k, k), dtype=np.int8)
    ws = (rng.random(M if per_channel else 1, dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    bias = rng.integers(-1000, 1000, M).astype(np.int32)
    return x, w, ws, bias


def test_noalloc_matches_regular_entry_point_twice(zb, ctx, oracle):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(2024)
    cases = [
        dict(N=2, C=16, H=12, W=11, M=24, k=3, group=1, xdt=I8, per_channel=True, pads=(1, 1, 1, 1), stride=(1, 1), act="relu", x_zp=0, y_zp=0),
        dict(N=3, C=8, H=9, W=9, M=8, k=3, group=8, xdt=U8, per_channel=False, pads=(0, 1, 1, 0), stride=(2, 2), act=None, x_zp=128, y_zp=3),
        # per-channel weight zero points: the second half of the shared array
        dict(N=1, C=6, H=7, W=8, M=10, k=3, group=1, xdt=I8, per_channel=True, pads=(1, 0, 0, 1), stride=(1, 1), act="relu6", x_zp=-5, y_zp=-2),
    ]
    for c in cases:                                     # two calls in a row on the same shared array
        x, w, ws, bias = _case(rng, c["N"], c["C"], c["H"], c["W"], c["M"], c["k"], c["group"], c["xdt"], c["per_channel"])
        wz = None if c["x_zp"] == 0 else rng.integers(-2, 3, ws.size).astype(np.int32)
        kw = dict(bias=bias, stride=c["stride"], pads=c["pads"], dilations=(1, 1), group=c["group"], activation=c["act"])
        want = ctx.qlinearconv(x, 0.02, c["x_zp"], w, ws, wz, 0.4, c["y_zp"], y_dtype=I8, **kw)
        xd, wd, bd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda()
        yd = torch.full(want.shape, 77, dtype=torch.int8, device="cuda")
        torch.cuda.synchronize()
        zb.qlinearconv_noalloc(xd, 0.02, c["x_zp"], wd, ws, wz, 0.4, c["y_zp"], yd, stream=torch.cuda.current_stream().cuda_stream,
                               **dict(kw, bias=bd))
        torch.cuda.synchronize()
        assert np.array_equal(yd.cpu().numpy(), want)
        assert np.array_equal(want, oracle.qlinearconv(x, 0.02, c["x_zp"], w, ws, wz, 0.4, c["y_zp"], y_dtype=I8, **kw))


def test_noalloc_rejects_what_it_cannot_hold(zb):
    torch = pytest.importorskip("torch")
    x = torch.zeros((1, 1, 1, 1), dtype=torch.int8, device="cuda")
    w = torch.zeros((4097, 1, 1, 1), dtype=torch.int8, device="cuda")
    y = torch.zeros((1, 4097, 1, 1), dtype=torch.int8, device="cuda")
    with pytest.raises(zb.ZantError) as e:
        zb.qlinearconv_noalloc(x, 0.1, 0, w, [0.1], None, 0.1, 0, y)
    assert e.value.name == "TooLarge"
    host_w = np.zeros((4, 1, 1, 1), np.int8)             # host buffers are refused: nothing is staged
    y4 = torch.zeros((1, 4, 1, 1), dtype=torch.int8, device="cuda")
    with pytest.raises(zb.ZantError) as e:
        zb.qlinearconv_noalloc(x, 0.1, 0, host_w, [0.1], None, 0.1, 0, y4)
    assert e.value.name == "InvalidInput"


def test_noalloc_refuses_a_capturing_stream(zb):
    """Every call copies its constants from host buffers, which a captured graph would re-read at each replay:
    the entry point refuses a stream that is being captured, and works again once the capture has ended."""
    torch = pytest.importorskip("torch")
    x = torch.ones((1, 2, 4, 4), dtype=torch.int8, device="cuda")
    w = torch.ones((3, 2, 1, 1), dtype=torch.int8, device="cuda")
    y = torch.zeros((1, 3, 4, 4), dtype=torch.int8, device="cuda")
    dummy = torch.zeros(16, device="cuda")
    zb.qlinearconv_noalloc(x, 1.0, 0, w, [1.0], None, 1.0, 0, y)          # first call on the device: before any capture
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s, capture_error_mode="thread_local"):
        dummy.add_(1.0)
        with pytest.raises(zb.ZantError) as e:
            zb.qlinearconv_noalloc(x, 1.0, 0, w, [1.0], None, 1.0, 0, y, stream=torch.cuda.current_stream().cuda_stream)
        assert e.value.name == "Unsupported"
    torch.cuda.synchronize()
    y.zero_()
    zb.qlinearconv_noalloc(x, 1.0, 0, w, [1.0], None, 1.0, 0, y)
    torch.cuda.synchronize()
    assert int(y.sum()) == 2 * 3 * 16
