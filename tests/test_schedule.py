"""The device-side work schedule of the tensor-core kernel, walked on the host (no GPU needed):
every K block of every tile is covered exactly once, whatever mix of whole tiles, uniform split-K
slices and stream-K runs a launch uses."""
import ctypes

import pytest

CASES = [
    # dtype, orient, bn, split_k, m, n, k
    (0, 1, 256, 1, 4096, 4096, 4096),      # 512 tiles on 148 CTAs: stream-K head of 68 tiles
    (0, 1, 256, 1, 1536, 4096, 4096),      # 192 tiles: head of 44
    (0, 1, 256, 1, 2048, 4096, 4096),      # 256 tiles: remainder 108 > half a wave, no head
    (0, 0, 64, 1, 1275, 1270, 1096),       # ragged edges, K tail inside a K block
    (0, 1, 128, 4, 128, 4096, 4096),       # uniform split-K, one unit per CTA
    (0, 1, 16, 8, 8, 4096, 14336),         # decode shape, 8 slices
    (0, 0, 32, 2, 700, 1000, 4096),        # more units than CTAs with split-K
    (0, 5, 256, 1, 4096, 4096, 4096),      # 256-row tiles
    (0, 4, 192, 1, 3000, 1100, 2048),
    (1, 1, 128, 1, 1300, 2100, 2048),      # INT8: 128 elements per K block
    (1, 0, 256, 2, 512, 6144, 4096),
    (0, 1, 64, 3, 40, 200, 640),           # odd slice count on a small problem
]


@pytest.mark.parametrize("dtype,orient,bn,split_k,m,n,k", CASES)
def test_schedule_covers_every_k_block_once(api, dtype, orient, bn, split_k, m, n, k):
    L = api.lib()
    L.mp_debug_schedule.argtypes = [ctypes.c_int] * 8 + [ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                                         ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    count = ctypes.c_int(0)
    info = (ctypes.c_int * 8)()
    assert L.mp_debug_schedule(dtype, orient, bn, 0, split_k, m, n, k, None, 0, ctypes.byref(count), info) == 0
    buf = (ctypes.c_int * (8 * count.value))()
    assert L.mp_debug_schedule(dtype, orient, bn, 0, split_k, m, n, k, buf, count.value, ctypes.byref(count), info) == 0
    grid, tiles, kb_total, ws_slices, sk_tiles, xm, helpers, S = list(info)
    units = [tuple(buf[8 * i: 8 * i + 8]) for i in range(count.value)]
    assert 1 <= grid <= 148 and xm == (2 if orient >= 4 else 1)
    rows = 128 * xm
    P, Q = (m, n) if orient in (0, 4) else (n, m)
    tiles_p, tiles_q = -(-P // rows), -(-Q // bn)
    assert tiles == tiles_p * tiles_q
    assert kb_total == -(-k // (128 if dtype == 1 else 64))

    per_tile = {}
    per_cta = {}
    for (cta, tile, tp, tq, kb0, kb1, sl, ns) in units:
        assert 0 <= cta < grid and 0 <= tile < tiles and 0 <= tp < tiles_p and 0 <= tq < tiles_q
        assert 0 <= kb0 < kb1 <= kb_total and 0 <= sl < ns
        per_tile.setdefault(tile, []).append((kb0, kb1, sl, ns, tp, tq, cta))
        per_cta.setdefault(cta, []).append(tile)
    assert sorted(per_tile) == list(range(tiles))                     # every tile is scheduled
    coords = set()
    for tile, parts in per_tile.items():
        parts.sort()
        assert parts[0][0] == 0 and parts[-1][1] == kb_total          # K covered from end to end ...
        for a, b in zip(parts, parts[1:]):
            assert a[1] == b[0]                                       # ... without gap or overlap
        ns = parts[0][3]
        assert len(parts) == ns and [p[2] for p in parts] == list(range(ns))   # slices numbered in K order
        assert len({(p[4], p[5]) for p in parts}) == 1                # one tile, one place in the output
        coords.add((parts[0][4], parts[0][5]))
        if ns > 1:
            assert ns <= ws_slices <= 31                              # the scratch has a slot for every slice
            assert len({p[6] for p in parts}) == ns                   # contributors are different CTAs
        if xm == 2:
            assert ns == 1
    assert len(coords) == tiles                                       # distinct tiles write distinct outputs
    if sk_tiles:
        assert S == 1 and 2 * sk_tiles <= grid and (tiles - sk_tiles) % grid == 0
        assert all(per_tile[t][0][3] >= 1 for t in range(sk_tiles))
        assert not helpers
    if helpers:
        assert count.value <= grid                                    # helping needs every unit running at once
    # balance: no CTA carries more than one whole tile (in K blocks) above the average
    load = {c: 0 for c in range(grid)}
    for (cta, tile, tp, tq, kb0, kb1, sl, ns) in units:
        load[cta] += kb1 - kb0
    avg = sum(load.values()) / grid
    assert max(load.values()) <= avg + kb_total


def test_schedule_rejects_bad_arguments(api):
    L = api.lib()
    L.mp_debug_schedule.argtypes = [ctypes.c_int] * 8 + [ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                                         ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    count = ctypes.c_int(0)
    assert L.mp_debug_schedule(2, 0, 128, 0, 1, 64, 64, 64, None, 0, ctypes.byref(count), None) == 1     # FP32 has no tile schedule
    assert L.mp_debug_schedule(0, 0, 100, 0, 1, 64, 64, 64, None, 0, ctypes.byref(count), None) == 1     # bn % 16
    assert L.mp_debug_schedule(0, 0, 128, 0, 1, 64, 64, 64, None, 0, None, None) == 1
