"""ctypes front-end of the CPU checker plus a numpy restatement for small cases.

TEST INFRASTRUCTURE: only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark import this module.  The product never does.

Every function follows the reference's host check loop
(moonpoly/core/moonpoly_gemm.cu:1610-1617): A row-major [m,k], B column-major
[k,n] (stored [n,k]), C column-major [m,n] (stored [n,m]); fp32 accumulation in
ascending k; `alpha*acc + beta*C` rounded to nearest in the output type.
Arrays are exchanged in *storage* order, i.e. B as an [n,k] array and C as an
[n,m] array.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile libmp_oracle.so beside this file (gcc, a second or two)."""
    so = os.path.join(_HERE, "libmp_oracle.so")
    src = os.path.join(_HERE, "mp_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libmp_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libmp_oracle.so")
        if not os.path.exists(so):
            build()
        _LIB = ctypes.CDLL(so)
    return _LIB


def _p(a: np.ndarray | None):
    if a is None:
        return ctypes.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def host_threads() -> int:
    return os.cpu_count() or 1


# --------------------------------------------------------------------------
# C-backed oracles
# --------------------------------------------------------------------------

def gemm_f16_rcc(A, B_nk, alpha=1.0, beta=0.0, C_nm=None, threads=None, f64acc=False):
    """A [m,k] f16, B_nk [n,k] f16 -> C_nm [n,m] f16 (column-major C of shape [m,n])."""
    A = np.ascontiguousarray(A, dtype=np.float16)
    B_nk = np.ascontiguousarray(B_nk, dtype=np.float16)
    m, k = A.shape
    n, k2 = B_nk.shape
    assert k == k2
    out = np.zeros((n, m), np.float16) if C_nm is None else np.array(C_nm, np.float16, order="C")
    fn = lib().orc_gemm_f16_rcc_f64acc if f64acc else lib().orc_gemm_f16_rcc
    fn(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), _p(A), _p(B_nk), _p(out),
       ctypes.c_float(alpha), ctypes.c_float(beta), ctypes.c_int(threads or host_threads()))
    return out


def gemm_f32_rcc(A, B_nk, alpha=1.0, beta=0.0, C_nm=None, threads=None):
    A = np.ascontiguousarray(A, dtype=np.float32)
    B_nk = np.ascontiguousarray(B_nk, dtype=np.float32)
    m, k = A.shape
    n, _ = B_nk.shape
    out = np.zeros((n, m), np.float32) if C_nm is None else np.array(C_nm, np.float32, order="C")
    lib().orc_gemm_f32_rcc(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), _p(A), _p(B_nk),
                           _p(out), ctypes.c_float(alpha), ctypes.c_float(beta),
                           ctypes.c_int(threads or host_threads()))
    return out


def gemm_i8_rcc(A, B_nk, ialpha=1, ibeta=0, C_nm=None, threads=None):
    A = np.ascontiguousarray(A, dtype=np.int8)
    B_nk = np.ascontiguousarray(B_nk, dtype=np.int8)
    m, k = A.shape
    n, _ = B_nk.shape
    out = np.zeros((n, m), np.int32) if C_nm is None else np.array(C_nm, np.int32, order="C")
    lib().orc_gemm_i8_rcc(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), _p(A), _p(B_nk),
                          _p(out), ctypes.c_int(ialpha), ctypes.c_int(ibeta),
                          ctypes.c_int(threads or host_threads()))
    return out


def scaled_mm_i8(A, B_nk, a_scales, b_scales, bias=None, out_bf16=False, threads=None):
    """A [M,K] i8, B_nk [N,K] i8, scales f32 (size 1 or M / N) -> out [M,N] row-major.

    fp16 output is returned as float16; bfloat16 output as its uint16 bit pattern.
    `bias` is float16 (or uint16 bf16 bits when out_bf16)."""
    A = np.ascontiguousarray(A, dtype=np.int8)
    B_nk = np.ascontiguousarray(B_nk, dtype=np.int8)
    M, K = A.shape
    N, _ = B_nk.shape
    a_scales = np.ascontiguousarray(a_scales, dtype=np.float32).reshape(-1)
    b_scales = np.ascontiguousarray(b_scales, dtype=np.float32).reshape(-1)
    assert a_scales.size in (1, M) and b_scales.size in (1, N)
    out = np.zeros((M, N), np.uint16 if out_bf16 else np.float16)
    if bias is not None:
        bias = np.ascontiguousarray(bias).reshape(-1)
        assert bias.size == N and bias.dtype == (np.uint16 if out_bf16 else np.float16)
    lib().orc_scaled_mm_i8(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), _p(A), _p(B_nk),
                           _p(a_scales), ctypes.c_int(int(a_scales.size == 1)),
                           _p(b_scales), ctypes.c_int(int(b_scales.size == 1)),
                           _p(bias), _p(out), ctypes.c_int(int(out_bf16)),
                           ctypes.c_int(threads or host_threads()))
    return out


def linear_f16(X, W, threads=None):
    """Linear(X[M,K], W[N,K]) -> Y[M,N] through the RCC remap (moonpoly_gemm.cu:41-44)."""
    X = np.ascontiguousarray(X, dtype=np.float16)
    W = np.ascontiguousarray(W, dtype=np.float16)
    M, K = X.shape
    N, _ = W.shape
    Y = np.zeros((M, N), np.float16)
    lib().orc_linear_f16(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), _p(X), _p(W), _p(Y),
                         ctypes.c_int(threads or host_threads()))
    return Y


def linear_bias(X, W, bias=None, bf16=False, threads=None):
    """Linear(X[M,K], W[N,K]) (+ bias[N]) -> Y[M,N], bias added in the output type after the rounding of the GEMM.
    fp16 arrays, or (bf16=True) uint16 arrays holding bfloat16 bit patterns; returns the same kind."""
    dt = np.uint16 if bf16 else np.float16
    X = np.ascontiguousarray(X, dtype=dt)
    W = np.ascontiguousarray(W, dtype=dt)
    M, K = X.shape
    N, _ = W.shape
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=dt).reshape(-1)
        assert bias.size == N
    Y = np.zeros((M, N), dt)
    lib().orc_linear_bias(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), _p(X), _p(W), _p(bias), _p(Y),
                          ctypes.c_int(int(bf16)), ctypes.c_int(threads or host_threads()))
    return Y


def twin_gemm_f16(A, B_nk, split_n, alpha=1.0, beta=0.0, C_nm=None, threads=None):
    A = np.ascontiguousarray(A, dtype=np.float16)
    B_nk = np.ascontiguousarray(B_nk, dtype=np.float16)
    m, k = A.shape
    n, _ = B_nk.shape
    out = np.zeros((n, m), np.float16) if C_nm is None else np.array(C_nm, np.float16, order="C")
    lib().orc_twin_gemm_f16(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), ctypes.c_int(split_n),
                            _p(A), _p(B_nk), _p(out), ctypes.c_float(alpha), ctypes.c_float(beta),
                            ctypes.c_int(threads or host_threads()))
    return out


# --------------------------------------------------------------------------
# numpy restatements (small cases; cross-check of the C code)
# --------------------------------------------------------------------------

def np_gemm_rcc(A, B_nk, alpha=1.0, beta=0.0, C_nm=None, out_dtype=None):
    """Sequential fp32 accumulation in ascending k, vectorised over outputs only."""
    out_dtype = out_dtype or A.dtype
    if A.dtype == np.int8:
        acc = A.astype(np.int32) @ B_nk.astype(np.int32).T          # exact
        r = np.int32(alpha) * acc
        if beta != 0:
            r = r + np.int32(beta) * C_nm.T.astype(np.int32)
        return np.ascontiguousarray(r.T.astype(np.int32))
    m, k = A.shape
    n = B_nk.shape[0]
    a32 = A.astype(np.float32)
    b32 = B_nk.astype(np.float32)
    acc = np.zeros((m, n), np.float32)
    for kk in range(k):
        acc = (acc + (a32[:, kk:kk + 1] * b32[:, kk][None, :]).astype(np.float32)).astype(np.float32)
    r = np.float32(alpha) * acc
    if beta != 0:
        r = (r + np.float32(beta) * C_nm.T.astype(np.float32)).astype(np.float32)
    return np.ascontiguousarray(r.T.astype(out_dtype))


def bf16_bits_from_f32(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def f32_from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def np_scaled_mm(A, B_nk, a_scales, b_scales, bias=None, out_bf16=False):
    acc = A.astype(np.int32) @ B_nk.astype(np.int32).T
    sa = np.asarray(a_scales, np.float32).reshape(-1, 1)
    sb = np.asarray(b_scales, np.float32).reshape(1, -1)
    t0 = (acc.astype(np.float32) * sb).astype(np.float32)
    t1 = (sa * t0).astype(np.float32)
    if not out_bf16:
        h = t1.astype(np.float16)
        if bias is not None:
            h = (h.astype(np.float32) + np.asarray(bias, np.float16).astype(np.float32).reshape(1, -1)).astype(np.float16)
        return h
    h = bf16_bits_from_f32(t1)
    if bias is not None:
        s = f32_from_bf16_bits(h) + f32_from_bf16_bits(np.asarray(bias, np.uint16)).reshape(1, -1)
        h = bf16_bits_from_f32(s.astype(np.float32))
    return h
