"""Host-side launch-shape rules of the streaming kernel (token split, cluster K split) and of the FP32 tile kernel,
through the library's test aids; no GPU needed (the rules use the SM count of the cost model, 148)."""
import ctypes

import pytest

from moonpoly_b200 import api


def _stream(dtype, m, n, k):
    out = (ctypes.c_int * 4)()
    assert api.lib().mp_debug_stream_launch(dtype, m, n, k, out) == 0
    return tuple(out)          # row CTAs, K parts, token parts, grid


def _f32(m, n, k):
    out = (ctypes.c_int * 3)()
    assert api.lib().mp_debug_f32_tile_launch(m, n, k, out) == 0
    return tuple(out)          # rows per CTA, K parts, grid


def test_streaming_kernel_launch_shapes_on_the_shapes_the_rules_were_measured_on():
    F, I = api.MP_FP16, api.MP_INT8
    assert _stream(F, 8, 4096, 4096) == (296, 1, 1, 296)            # enough rows: two whole-K CTAs per SM
    assert _stream(F, 32, 4096, 4096) == (296, 1, 1, 296)           # a token split never pays on a full grid
    assert _stream(F, 1, 1024, 28672) == (64, 4, 1, 256)            # few rows, long K: 16-row blocks x 4 K parts
    assert _stream(F, 8, 1024, 28672) == (64, 4, 1, 256)
    assert _stream(F, 1, 2048, 28672) == (148, 2, 1, 296)
    assert _stream(F, 1, 1024, 8192) == (128, 1, 1, 128)            # K too short for a split to pay
    assert _stream(F, 32, 1024, 8192) == (128, 1, 2, 256)           # ... but more than 8 tokens split in two
    assert _stream(F, 8, 2048, 8192) == (148, 1, 1, 148)
    assert _stream(I, 16, 1024, 28672) == (64, 2, 2, 256)           # INT8: half the bytes per row, 2 K parts
    # both mappings give the same shape (the wide side is streamed whichever operand it is)
    assert _stream(F, 1024, 8, 28672) == _stream(F, 8, 1024, 28672)


def test_streaming_kernel_launch_shape_invariants():
    for dtype, elt in ((api.MP_FP16, 2), (api.MP_INT8, 1)):
        for r in (1, 7, 64, 500, 1024, 1280, 2048, 2368, 2560, 4096, 28672):
            for t in (1, 8, 9, 16, 33, 64):
                for k in (16, 1024, 4096, 8192, 28672, 65536):
                    rows, ks, ts, grid = _stream(dtype, t, r, k)
                    assert grid == rows * ks * ts and rows >= 1
                    assert ks in (1, 2, 4, 8) and 1 <= ts <= (t + 7) // 8
                    if ks > 1:
                        assert k * elt >= 4096 * ks                 # every warp keeps a full batch of loads
                        assert rows * ks <= 2 * 148                 # at most two CTAs per SM
                        assert r < 8 * 2 * 148                      # only weights that cannot fill the GPU by rows
                    if ts > 1:
                        assert t > 8


def test_fp32_tile_kernel_launch_shapes():
    assert _f32(37, 1024, 1024) == (32, 4, 128)                     # the config shape: 32 row blocks x 4 K parts
    assert _f32(1024, 37, 1024) == (32, 4, 128)
    assert _f32(37, 4096, 1024) == (32, 1, 128)
    assert _f32(37, 256, 1024) == (32, 8, 64)
    assert _f32(64, 256, 256) == (32, 2, 16)                        # never more parts than 128-float chunks of K
    for r in (9, 40, 100, 1000, 5000, 30000):
        for k in (4, 128, 1000, 4096):
            rows, ks, grid = _f32(20, r, k)
            assert rows == 32 and ks in (1, 2, 4, 8) and ks <= max(1, (k + 127) // 128)
            assert grid == (max(r, 20) + 31) // 32 * ks


def test_launch_rule_aids_reject_bad_arguments():
    out = (ctypes.c_int * 4)()
    assert api.lib().mp_debug_stream_launch(api.MP_FP32, 8, 1024, 1024, out) != 0
    assert api.lib().mp_debug_stream_launch(api.MP_FP16, 0, 1024, 1024, out) != 0
    assert api.lib().mp_debug_f32_tile_launch(37, 1024, 0, (ctypes.c_int * 3)()) != 0
