"""The C++ boundary: every function the reference's callers link to is exported with the reference's own mangled
name (namespace moonpoly, moonpoly::fp16::row_col_col and the fp32 / int8 cost namespaces), and the host-only
ones answer without a GPU."""
import ctypes
import os
import re
import subprocess

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
PKG = os.path.join(ROOT, "moonpoly-dev_b200")
LIB = os.path.join(PKG, "libmoonpoly_gemm.so")


def exported():
    out = subprocess.run(["nm", "-DC", "--defined-only", LIB], capture_output=True, text=True, check=True).stdout
    return out


def declared_functions(header):
    """Function names declared at namespace scope in a header, qualified by their namespaces."""
    text = open(os.path.join(PKG, "host", header)).read()
    text = re.sub(r"//.*", "", text)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    names, stack, stmt = [], [], ""
    for ch in text:
        if ch == "{":
            m = re.search(r"namespace\s+(\w+)\s*$", stmt)
            stack.append(m.group(1) if m else None)
            stmt = ""
        elif ch == "}":
            stack.pop()
            stmt = ""
        elif ch == ";":
            if None not in stack:
                m = re.search(r"(\w+)\s*\([^()]*\)\s*$", stmt.strip(), flags=re.S)
                if m and not stmt.strip().startswith(("struct", "enum", "const int num")):
                    names.append("::".join(stack + [m.group(1)]))
            stmt = ""
        else:
            stmt += ch
    return names


def test_every_declared_cxx_function_is_exported():
    syms = exported()
    want = []
    for h in ("moonpoly.cuh", "candidates.cuh", "moonpoly_cost.cuh"):
        want += declared_functions(h)
    assert len(want) >= 45, want
    for must in ("moonpoly::run_fp16_gemm", "moonpoly::fp16::row_col_col::run_explicit_neighborhood_gemm",
                 "moonpoly::fp16::row_col_col::gemm_splitk_cost_model", "moonpoly::int8::row_col_col::cutlass_gemm_predict",
                 "moonpoly::fp32::simt::row_col_col::gemm_cost_model"):
        assert must in want
    # the five StreamK workspace getters are declared through a macro in the header: name them here
    want = [w for w in want if not w.split("::")[-1].startswith("_")]
    want += [f"moonpoly::get_fp16_p{p}_streamk_workspace_size_row_col_col" for p in (40, 42, 43, 44, 66)]
    missing = [w for w in want if (w + "(") not in syms]
    assert not missing, missing
    assert "moonpoly::fp16::row_col_col::num_gemm_primary" in syms


def _sym(L, namespaces, name, args, restype, argtypes):
    """Itanium-mangled lookup: _ZN<len><ns>...<len><name>E<args> (args: 'v' or a run of 'i')."""
    mangled = "_ZN" + "".join(f"{len(x)}{x}" for x in list(namespaces) + [name]) + "E" + args
    f = getattr(L, mangled)
    f.restype, f.argtypes = restype, argtypes
    return f


def test_candidates_and_cost_api_answer_on_the_host():
    L = ctypes.CDLL(LIB)
    ci, cf = ctypes.c_int, ctypes.c_float
    ns = ("moonpoly", "fp16", "row_col_col")
    is_explicit = _sym(L, ns, "is_explicit_neighborhood_pid", "i", ctypes.c_bool, [ci])
    is_elite = _sym(L, ns, "is_paper_elite_fp16_pid", "i", ctypes.c_bool, [ci])
    count = _sym(L, ns, "paper_elite_fp16_kernel_count", "v", ci, [])
    pids = _sym(L, ns, "paper_elite_fp16_pids", "v", ctypes.POINTER(ci), [])
    align = _sym(L, ns, "explicit_neighborhood_alignment", "i", ci, [ci])
    cost = _sym(L, ns, "gemm_cost_model", "iiii", cf, [ci, ci, ci, ci])
    split = _sym(L, ns, "gemm_splitk_cost_model", "iiiii", cf, [ci, ci, ci, ci, ci])
    red = _sym(L, ns, "gemm_reduction_cost_model", "iiiii", cf, [ci, ci, ci, ci, ci])
    predict = _sym(L, ns, "cutlass_gemm_predict", "iii", ci, [ci, ci, ci])

    # generated/fp16/rcc/candidates.cu:35-65
    assert [is_explicit(p) for p in (89, 90, 205, 206, 215, 216, 321, 322, 399, 400, 439, 440)] == \
        [False, True, True, False, False, True, True, False, False, True, True, False]
    assert count() == 45 and [pids()[i] for i in (0, 39, 40, 44)] == [0, 39, 400, 439]
    assert is_elite(413) and not is_elite(401) and not is_elite(40)
    assert align(114) == 4 and align(91) == 8 and align(400) == 8 and align(5) == 1
    # cost API: feature order (ims tiled by pm = RCC n, ins tiled by pn = RCC m)
    c1 = cost(16, 4096, 4096, 8)
    assert 0.0 < c1 < 1.0
    assert red(16, 4096, 4096, 7, 1) == 0.0 and red(16, 4096, 4096, 7, 4) > 0.0
    assert abs(split(16, 4096, 4096, 7, 1) - cost(16, 4096, 4096, 7)) < 1e-9
    assert split(16, 4096, 4096, 7, 4) > 0.0
    best = predict(16, 4096, 4096)
    assert 0 <= best < 40
    assert all(cost(16, 4096, 4096, best) <= cost(16, 4096, 4096, p) + 1e-9 for p in range(40))
    for ns2, n_pids in ((("moonpoly", "fp32", "simt", "row_col_col"), 40), (("moonpoly", "int8", "row_col_col"), 46)):
        c = _sym(L, ns2, "gemm_cost_model", "iiii", cf, [ci, ci, ci, ci])
        s = _sym(L, ns2, "gemm_splitk_cost_model", "iiii", cf, [ci, ci, ci, ci])
        p = _sym(L, ns2, "cutlass_gemm_predict", "iii", ci, [ci, ci, ci])
        assert 0 <= p(37, 1024, 1024) < n_pids
        assert c(37, 1024, 1024, 0) > 0.0 and s(37, 1024, 4096, 2) > 0.0
