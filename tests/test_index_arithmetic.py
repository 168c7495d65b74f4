"""Index arithmetic of two shared-memory kernels, restated on the CPU and checked over many shapes.

The stem mode of the pointwise kernel (`z-ant_b200/csrc/tc_pw_nchw.cuh`: `pw_stem_plan`, the loader's bulk
copies, `pw_stem_builder`) and the rows-form depthwise kernel (`z-ant_b200/csrc/dwconv_q8.cuh`: the batch
sizes chosen in `run_qdwconv`, the loads and stores of `qdwconv3x3_rows_kernel`) address shared memory by
computed offsets.  These tests repeat that arithmetic in Python for grids of shapes and assert the
invariants the kernels rely on: every bulk copy starts on 16 bytes, is a multiple of 16 bytes long and
stays inside its buffer; every input row a builder reads was loaded; every load and store stays inside
its buffer (with the 16 bytes in front and behind that the kernels reserve); the one-multiplication
division by the output width is exact; only the first pixel of tap 0 and the last pixel of a tap can lie
outside the image.  No GPU is involved; the formulas must be kept in step with the kernels.
"""
import itertools

import pytest


def stem_plan(N, C, H, W, M, cs, pt, pl, pb, pr):
    OH = (H + pt + pb - 3) // cs + 1
    OW = (W + pl + pr - 3) // cs + 1
    if not (1 <= C <= 3) or not (1 <= M <= 64) or OH <= 0 or OW <= 0 or max(pt, pl, pb, pr) > 1:
        return None
    hw = OH * OW
    if W % 16 or OW % 16 or hw % 16 or hw > (1 << 24) or H * W > (1 << 24):
        return None
    if (OW - 4) * cs + 2 - pl + 2 * cs >= W or hw * OW >= (1 << 32):
        return None
    m_pad = 16 if M <= 16 else (32 if M <= 32 else 64)
    G = 128 // m_pad
    if hw < G * 64 or N * hw < 4096:
        return None
    tile_max = 256 * G
    px_tiles = (hw + tile_max - 1) // tile_max
    n_px = ((hw + px_tiles * G - 1) // (px_tiles * G) + 15) // 16 * 16
    tile_px = G * n_px
    rows_out = (tile_px + OW - 2) // OW + 1
    band = (rows_out - 1) * cs + 3
    raw = 16 + C * band * W + 16
    if raw > 40000:
        return None
    raw_bytes = (raw + 127) // 128 * 128
    return dict(OH=OH, OW=OW, hw=hw, G=G, px_tiles=px_tiles, n_px=n_px, tile_px=tile_px, band=band,
                raw_bytes=raw_bytes, magic=(1 << 32) // OW + 1)


STEM_GRID = [(C, cs, pt, pl, pb, pr, W, H, M)
             for C, cs, pt, pl, pb, pr in itertools.product((1, 3), (1, 2), (0, 1), (0, 1), (0, 1), (0, 1))
             for W in (32, 112, 224, 416) for H in (13, 64, 224) for M in (8, 32, 64)]


def test_stem_mode_offsets_stay_inside_their_buffers():
    checked = 0
    for C, cs, pt, pl, pb, pr, W, H, M in STEM_GRID:
        N = max(1, (4096 + H * W - 1) // (H * W)) * 2
        p = stem_plan(N, C, H, W, M, cs, pt, pl, pb, pr)
        if p is None:
            continue
        checked += 1
        OH, OW, hw, G, n_px, tile_px, band = p["OH"], p["OW"], p["hw"], p["G"], p["n_px"], p["tile_px"], p["band"]
        NX, nc = 4 * cs, n_px >> 4
        where = (C, cs, pt, pl, pb, pr, W, H, M)
        for ti in range(p["px_tiles"]):
            p0 = ti * tile_px
            assert (p0 * p["magic"]) >> 32 == p0 // OW, where
            oh_a, oh_b = p0 // OW, min(OH - 1, (min(hw, p0 + tile_px) - 1) // OW)
            ih_lo = oh_a * cs - pt
            r0, r1 = max(ih_lo, 0), min(H, oh_b * cs - pt + 3)
            assert r1 > r0, where
            for c in range(C):                                          # the loader's bulk copies
                dst, nbytes = 16 + (c * band + (r0 - ih_lo)) * W, (r1 - r0) * W
                assert dst % 16 == 0 and nbytes % 16 == 0 and dst + nbytes <= p["raw_bytes"] and r1 - 1 - ih_lo < band, where
            for pg, ci in itertools.product(range(G), range(16)):       # a builder lane's chunk
                pp = p0 + pg * n_px + 16 * ci
                assert (pp * p["magic"]) >> 32 == pp // OW, where
                oy = pp // OW
                ox = pp - oy * OW
                if not (ci < nc and pp < hw):
                    continue
                assert ox + 16 <= OW, where                             # the 16 pixels lie in one output row
                row0 = oy * cs - pt
                for kh in range(3):
                    iy = row0 + kh
                    if not 0 <= iy < H:
                        continue
                    assert r0 <= iy < r1, where                         # the row was loaded
                    for c in range(C):
                        ad = 16 + (row0 - ih_lo) * W + ox * cs + c * band * W + kh * W
                        assert ad % 16 == 0 and ad - 4 >= 0 and ad + 4 * NX + 4 <= p["raw_bytes"], where
                for kw in range(3):
                    first, prev, last = ox * cs + kw - pl, (ox + 14) * cs + kw - pl, (ox + 15) * cs + kw - pl
                    assert prev < W and first >= -1 and (first >= 0 or kw == 0), where
                    room = W - 15 * cs - (ox * cs - pl)
                    assert (kw >= room) == (last >= W), where
    assert checked > 200


def test_rows_form_depthwise_batches_and_offsets():
    configs = 0
    for S, widths in ((1, (7, 14, 28)), (2, (14, 28))):
        for W, H in itertools.product(widths, range(1, 80)):
            OH, OW = (H, W) if S == 1 else ((H + 1) // 2, W // 2)
            if OH > 64:
                continue
            P, PO = H * W, OH * OW
            unit = 16
            while unit > 1 and (P * (unit // 2)) % 16 == 0 and (PO * (unit // 2)) % 16 == 0:
                unit //= 2
            PB = 256 // OH // unit * unit
            if PB < unit:
                continue
            buf, out = PB * P, PB * PO
            in_stride, out_stride = (buf + 32 + 127) // 128 * 128, (out + 127) // 128 * 128
            if 3 * in_stride + 2 * out_stride + 32 > 48 * 1024:
                continue
            configs += 1
            where = (S, W, H, PB)
            assert buf % 16 == 0 and out % 16 == 0 and PB * OH <= 256, where
            NA = (W + 2 + 3) // 4
            for pl in (0, PB - 1):
                for r in range(OH):
                    for kr in range(3):
                        iy = S * r + kr - 1
                        if 0 <= iy < H:
                            sb = pl * P + iy * W - 1
                            lo = 16 + (sb & ~3)                          # offset from the buffer's start: 16 bytes lie in front of the planes
                            assert lo >= 0 and lo + 4 * (NA + 1) <= in_stride, where
                    for x in range(OW):
                        j, o = (S * x) // 4, (S * x) % 4
                        assert j < NA and (o == 0 or j + 1 <= NA) and S * x + 2 <= W + 1, where
                    assert pl * PO + r * OW + OW <= out, where
    assert configs > 100
