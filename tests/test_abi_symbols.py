"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares."""
import ctypes
import glob
import os
import re

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names |= set(re.findall(r"\b(mp_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(api):
    L = ctypes.CDLL(api.LIB_PATH)
    syms = declared_symbols()
    assert len(syms) >= 18
    for s in syms:
        assert hasattr(L, s), f"{s} declared in include/ but not exported"


def test_host_only_queries_need_no_gpu(api):
    assert api.version().startswith("moonpoly-b200")
    tile, align = api.pid_info(api.MP_FP16, 0)
    assert tile[2] == 64 and align == 8
    assert api.elite_fp16_pids()[-5:] == [400, 407, 413, 425, 439] and len(api.elite_fp16_pids()) == 45
    assert api.get_int8_scaled_mm_kernel_config(0)[3] == 16


def test_scratch_growth_rule_matches_the_buffer_layout(api):
    """The library's per-stream split-K scratch is a counter area followed by the partial sums.  The counter area
    keeps the size it was created with, so capacity must be tested against that size, not against what the current
    call asks for."""
    must_grow = api.lib().mp_debug_scratch_must_grow
    must_grow.argtypes = [ctypes.c_size_t] * 4
    KB, MB = 1 << 10, 1 << 20
    assert must_grow(8 * MB + 64 * KB, 64 * KB, 64 * KB, 8 * MB) == 0          # exactly fits
    assert must_grow(8 * MB + 64 * KB, 64 * KB, 64 * KB, 8 * MB + 1) == 1
    assert must_grow(8 * MB + 64 * KB, 64 * KB, 128 * KB, 1 * MB) == 1         # more counters than the buffer has
    # a buffer created by a many-tile call has a 256 KB counter area: partials start behind it
    have = 256 * KB + 8 * MB
    assert must_grow(have, 256 * KB, 64 * KB, 8 * MB) == 0
    assert must_grow(have, 256 * KB, 64 * KB, 8 * MB + 100 * KB) == 1          # would fit behind 64 KB, not behind 256 KB
    for want in (64 * KB, 256 * KB):
        for part in range(0, 9 * MB, 512 * KB):
            fits = max(256 * KB, want) + part <= have
            assert must_grow(have, 256 * KB, want, part) == (0 if fits else 1)


def test_workspace_size_covers_the_fallback_tiles_of_the_streaming_pids(api):
    """pids 1100 / 1101 fall back to a narrow tensor tile whose orientation follows the problem; the reported
    workspace must cover that launch for every (m, n), in both orientations."""
    sched = api.lib().mp_debug_schedule
    info = (ctypes.c_int * 8)()
    count = ctypes.c_int()
    k, split = 2048, 2
    for pid in (1100, 1101):
        for m in (1, 9, 65, 70, 130, 200, 300):
            for n in (1, 9, 65, 70, 130, 200, 300):
                reported = api.workspace_size(api.MP_FP16, pid, m, n, k, split)
                orient = 1 if m <= n else 0
                bn = 16 if pid == 1100 else min(64, max(16, (min(m, n) + 15) // 16 * 16))
                assert sched(api.MP_FP16, orient, bn, 0, split, m, n, k, None, 0, ctypes.byref(count), info) == 0
                tiles, slices = info[1], info[3]
                need = (tiles * 64 + 255) // 256 * 256 + tiles * slices * bn * 128 * 4
                assert reported >= need, (pid, m, n, reported, need)
