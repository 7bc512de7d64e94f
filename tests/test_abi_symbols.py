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
