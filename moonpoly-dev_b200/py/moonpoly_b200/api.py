"""Python host side above the C ABI of libmoonpoly_gemm.so.

Mirrors the reference's Python surface (pybind module `moonpoly` and dispatcher library
`moonpoly_ops`, moonpoly/core/moonpoly_gemm.cu:516-558 and :1784-1927): same function names,
argument meaning and error behaviour.  torch is used for device memory and streams only; every
computation goes through the C ABI with raw device pointers.  There is no CPU or torch fallback:
when the CUDA library cannot be loaded, importing the compute entry points raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

MP_FP16, MP_INT8, MP_FP32, MP_BF16 = 0, 1, 2, 3
MP_OK = 0
STATUS_NAMES = {0: "MP_OK", 1: "MP_ERR_INVALID_ARG", 2: "MP_ERR_LAYOUT", 3: "MP_ERR_UNALIGNED_K",
                4: "MP_ERR_BAD_PID", 5: "MP_ERR_WORKSPACE", 6: "MP_ERR_CUDA", 7: "MP_ERR_DEVICE",
                8: "MP_ERR_UNSUPPORTED"}

_PKG_ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
LIB_PATH = os.path.join(_PKG_ROOT, "libmoonpoly_gemm.so")


class Plan(ctypes.Structure):
    """Same fields as moonpoly::Fp16OnlinePlan (moonpoly/include/moonpoly.cuh:39-45)."""
    _fields_ = [("pattern", ctypes.c_int), ("pid", ctypes.c_int), ("split_k", ctypes.c_int),
                ("split_n", ctypes.c_int), ("estimated_ms", ctypes.c_float)]

    def __repr__(self):
        return (f"Plan(pattern={self.pattern}, pid={self.pid}, split_k={self.split_k}, "
                f"split_n={self.split_n}, estimated_ms={self.estimated_ms:.5f})")


class MoonpolyError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """Load libmoonpoly_gemm.so (built in-tree by `make -C moonpoly-dev_b200`); raise if absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `make -C {_PKG_ROOT}` "
                              "(there is no fallback implementation)")
        L = ctypes.CDLL(LIB_PATH)
        L.mp_last_error_string.restype = ctypes.c_char_p
        L.mp_version.restype = ctypes.c_char_p
        L.mp_launch_count.restype = ctypes.c_ulonglong
        vp, ci, cf, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
        L.mp_gemm.argtypes = [ci, ci, ci, ci, vp, ci, vp, ci, vp, ci, cf, cf, vp]
        L.mp_linear.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp]
        L.mp_gemm_rcc.argtypes = [ci, ci, ci, ci, vp, vp, vp, cf, cf, vp]
        L.mp_gemm_rcc_pid.argtypes = [ci, ci, ci, ci, ci, ci, vp, vp, vp, cf, cf, vp, sz, vp]
        L.mp_gemm_rcc_pid_static_scratch.argtypes = [ci, ci, ci, ci, ci, ci, vp, vp, vp, cf, cf, vp]
        L.mp_gemm_rcc_tile.argtypes = [ci, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp, cf, cf, vp]
        L.mp_workspace_size.argtypes = [ci, ci, ci, ci, ci, ci, ctypes.POINTER(sz)]
        L.mp_select_plan.argtypes = [ci, ci, ci, ci, ctypes.POINTER(Plan)]
        L.mp_pid_info.argtypes = [ci, ci, ctypes.POINTER(ci * 3), ctypes.POINTER(ci)]
        L.mp_cost_ms.argtypes = [ci, ci, ci, ci, ci, ci, ctypes.POINTER(cf)]
        L.mp_twin_gemm_fp16.argtypes = [ci, ci, ci, ci, vp, vp, vp, cf, cf, vp]
        L.mp_scaled_mm_i8.argtypes = [ci, ci, ci, vp, ci, vp, ci, vp, ci, vp, ci, vp, vp, ci, ci, vp]
        L.mp_scaled_mm_i8_tile.argtypes = [ci, ci, ci, ci, ci, ci, vp, ci, vp, ci, vp, ci, vp, ci, vp, vp, ci, ci, vp]
        L.mp_scaled_mm_predict.argtypes = [ci, ci, ci]
        L.mp_scaled_mm_config.argtypes = [ci, ctypes.POINTER(ci * 4)]
        L.mp_elite_fp16_pids.argtypes = [ctypes.POINTER(ci), ci]
        L.mp_device_status.argtypes = [vp, ctypes.POINTER(ci)]
        L.mp_linear_bias.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, vp]
        L.mp_linear_gather.argtypes = [ci, ci, ci, ci, vp, vp, ctypes.POINTER(vp), ci, ctypes.c_longlong, ctypes.c_longlong, vp]
        L.mp_peer_barrier.argtypes = [vp, ci, ci, ctypes.c_uint, ctypes.c_uint, vp]
        L.mp_peer_alloc.argtypes = [sz, ctypes.POINTER(vp), ctypes.c_char_p]
        L.mp_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.mp_peer_close.argtypes = [vp]
        L.mp_peer_free.argtypes = [vp]
        _lib = L
    return _lib


def _check(rc: int) -> None:
    if rc != MP_OK:
        raise MoonpolyError(rc, lib().mp_last_error_string().decode())


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return MP_FP16
    if t.dtype == torch.int8:
        return MP_INT8
    if t.dtype == torch.float32:
        return MP_FP32
    if t.dtype == torch.bfloat16:
        # moonpoly/core/moonpoly_gemm.cu:74-77
        raise ValueError("BF16 core GEMM has been removed; use FP16/FP32/INT8")
    raise ValueError(f"Unsupported data type {t.dtype}")


# ------------------------------------------------------------------------------------------------
# queries (host only)
# ------------------------------------------------------------------------------------------------
def version() -> str:
    return lib().mp_version().decode()


def num_sms() -> int:
    return lib().mp_num_sms()


def launch_count() -> int:
    return int(lib().mp_launch_count())


def reload_env() -> None:
    _check(lib().mp_reload_env())


def select_plan(dtype: int, m: int, n: int, k: int) -> Plan:
    """select_fp16_online_plan_row_col_col and its fp32 / int8 siblings, on RCC (m, n, k)."""
    p = Plan()
    _check(lib().mp_select_plan(dtype, m, n, k, ctypes.byref(p)))
    return p


def pid_info(dtype: int, pid: int):
    """([pm, pn, pk], alignment): get_gemm_shared_mem_* / get_gemm_alignment_*."""
    tile = (ctypes.c_int * 3)()
    align = ctypes.c_int()
    _check(lib().mp_pid_info(dtype, pid, ctypes.byref(tile), ctypes.byref(align)))
    return list(tile), align.value


def cost_ms(dtype: int, pid: int, split_k: int, m: int, n: int, k: int) -> float:
    v = ctypes.c_float()
    _check(lib().mp_cost_ms(dtype, pid, split_k, m, n, k, ctypes.byref(v)))
    return v.value


def elite_fp16_pids() -> list:
    n = lib().mp_elite_fp16_pids(None, 0)
    buf = (ctypes.c_int * n)()
    lib().mp_elite_fp16_pids(buf, n)
    return list(buf)


def workspace_size(dtype: int, pid: int, m: int, n: int, k: int, split_k: int = 2) -> int:
    v = ctypes.c_size_t()
    _check(lib().mp_workspace_size(dtype, pid, m, n, k, split_k, ctypes.byref(v)))
    return int(v.value)


def device_status(sync_stream=None) -> int:
    """Synchronise and return the device status word (raises MoonpolyError when non-zero)."""
    code = ctypes.c_int()
    rc = lib().mp_device_status(ctypes.c_void_p(0), ctypes.byref(code))
    _check(rc)
    return code.value


def predict_int8_scaled_mm_kernel(m: int, n: int, k: int) -> int:
    return lib().mp_scaled_mm_predict(m, n, k)


def get_int8_scaled_mm_kernel_config(kernel_id: int):
    out = (ctypes.c_int * 4)()
    _check(lib().mp_scaled_mm_config(kernel_id, ctypes.byref(out)))
    return tuple(out)


# ------------------------------------------------------------------------------------------------
# RCC entry points (device tensors)
# ------------------------------------------------------------------------------------------------
def _out_dtype(t: torch.Tensor) -> torch.dtype:
    return torch.int32 if t.dtype == torch.int8 else t.dtype


def gemm_rcc(a: torch.Tensor, b_nk: torch.Tensor, c_nm: Optional[torch.Tensor] = None, alpha: float = 1.0,
             beta: float = 0.0) -> torch.Tensor:
    """moonpoly_gemm(dtype, m, n, k, A,false, B,true, C,true, alpha, beta): a [m,k], b_nk [n,k]
    (= column-major [k,n]), returns c_nm [n,m] (= column-major [m,n])."""
    dt = _dtype_code(a)
    m, k = a.shape
    n = b_nk.shape[0]
    assert b_nk.shape[1] == k and a.is_contiguous() and b_nk.is_contiguous()
    if c_nm is None:
        c_nm = torch.empty((n, m), dtype=_out_dtype(a), device=a.device)
    _check(lib().mp_gemm(dt, m, n, k, _ptr(a), 0, _ptr(b_nk), 1, _ptr(c_nm), 1, alpha, beta, _stream(a)))
    return c_nm


def gemm_rcc_pid(a: torch.Tensor, b_nk: torch.Tensor, pid: int, split_k: int = 1,
                 c_nm: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
                 workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """run_moonpoly_selected_gemm_*_row_col_col_with_workspace on RCC operands."""
    dt = _dtype_code(a)
    m, k = a.shape
    n = b_nk.shape[0]
    if c_nm is None:
        c_nm = torch.empty((n, m), dtype=_out_dtype(a), device=a.device)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _check(lib().mp_gemm_rcc_pid(dt, pid, split_k, m, n, k, _ptr(a), _ptr(b_nk), _ptr(c_nm), alpha, beta,
                                 _ptr(workspace), ws_bytes, _stream(a)))
    return c_nm


def gemm_rcc_tile(a: torch.Tensor, b_nk: torch.Tensor, orient: int, bn: int, kc: int = 0, split_k: int = 1,
                  c_nm: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0) -> torch.Tensor:
    """Tuning entry: the tensor-core kernel with an explicit tile (see mp_gemm_rcc_tile)."""
    dt = _dtype_code(a)
    m, k = a.shape
    n = b_nk.shape[0]
    if c_nm is None:
        c_nm = torch.empty((n, m), dtype=_out_dtype(a), device=a.device)
    _check(lib().mp_gemm_rcc_tile(dt, orient, bn, kc, split_k, m, n, k, _ptr(a), _ptr(b_nk), _ptr(c_nm), alpha, beta,
                                  _stream(a)))
    return c_nm


def twin_gemm_fp16(a: torch.Tensor, b_nk: torch.Tensor, split_n: int, c_nm: Optional[torch.Tensor] = None,
                   alpha: float = 1.0, beta: float = 0.0) -> torch.Tensor:
    """run_fp16_pattern2_twin_gemm_row_col_col; invalid split_n / k raise ValueError as the
    reference throws std::invalid_argument."""
    m, k = a.shape
    n = b_nk.shape[0]
    if c_nm is None:
        c_nm = torch.empty((n, m), dtype=torch.float16, device=a.device)
    rc = lib().mp_twin_gemm_fp16(m, n, k, split_n, _ptr(a), _ptr(b_nk), _ptr(c_nm), alpha, beta, _stream(a))
    if rc == 1:
        raise ValueError(lib().mp_last_error_string().decode())
    _check(rc)
    return c_nm


# ------------------------------------------------------------------------------------------------
# the `moonpoly` / `moonpoly_ops` surface the vLLM Linear patch calls
# ------------------------------------------------------------------------------------------------
def _linear_checks(x: torch.Tensor, w: torch.Tensor) -> None:
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("A and B must be 2-D tensors")
    if x.shape[1] != w.shape[1]:
        raise ValueError("A and B must have the same K (A: [M,K], B: [N,K])")
    if not (x.is_cuda and w.is_cuda):
        raise ValueError("A and B must be CUDA tensors")
    if x.dtype != w.dtype:
        raise ValueError("A and B must have the same dtype")


def linear_bias(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y[M,N] = X[M,K] @ W[N,K]^T (+ bias[N]) in one launch, fp16 or bf16 (the reference adds the bias with a second
    kernel and serves fp16 only).  The bias is added in the output type after the GEMM's rounding, so the result is
    bit-identical to `linear(x, w) + bias`."""
    _linear_checks(x, w)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("linear_bias serves fp16 and bf16")
    x = x.contiguous()
    w = w.contiguous()
    M, K = x.shape
    N = w.shape[0]
    if bias is not None:
        if bias.dtype != x.dtype or bias.numel() != N or not bias.is_cuda:
            raise ValueError("bias must be a CUDA tensor of N elements in the input dtype")
        bias = bias.contiguous()
    y = torch.empty((M, N), dtype=x.dtype, device=x.device)
    _check(lib().mp_linear_bias(MP_FP16 if x.dtype == torch.float16 else MP_BF16, M, N, K, _ptr(x), _ptr(w), _ptr(bias),
                                _ptr(y), _stream(x)))
    return y


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """moonpoly.linear / moonpoly_ops.linear: Y[M,N] = X[M,K] @ W[N,K]^T on the current stream.  bf16 inputs, which
    the reference refuses (moonpoly/core/moonpoly_gemm.cu:74-77), are served here by the same tensor-core kernels."""
    _linear_checks(x, w)
    if x.dtype == torch.bfloat16:
        return linear_bias(x, w, None)
    x = x.contiguous()
    w = w.contiguous()
    dt = _dtype_code(x)
    M, K = x.shape
    N = w.shape[0]
    y = torch.empty((M, N), dtype=_out_dtype(x), device=x.device)
    _check(lib().mp_linear(dt, M, N, K, _ptr(x), _ptr(w), _ptr(y), _stream(x)))
    return y


def linear_cpp_selector(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """moonpoly_ops.linear_cpp_selector: the measured decode plans are part of the online
    selector here, so this is `linear` (non-fp16 input falls back to `linear` in the reference too)."""
    return linear(x, w)


def fp16_workspace_size(x: torch.Tensor, w: torch.Tensor, pid: int, split_k_slices: int = 2) -> int:
    M, K = x.shape
    N = w.shape[0]
    return workspace_size(MP_FP16, pid, N, M, K, 2 if split_k_slices <= 0 else split_k_slices)


def fp16_rcc_workspace_size(a: torch.Tensor, b_col: torch.Tensor, pid: int, split_k_slices: int = 2) -> int:
    m, k = a.shape
    n = b_col.shape[1]
    return workspace_size(MP_FP16, pid, m, n, k, 2 if split_k_slices <= 0 else split_k_slices)


def _check_workspace(workspace: Optional[torch.Tensor], need: int) -> None:
    # moonpoly/core/moonpoly_gemm.cu:383-398
    if need == 0:
        return
    if workspace is None or not workspace.is_cuda or workspace.dtype != torch.uint8 or not workspace.is_contiguous():
        raise ValueError("workspace must be a contiguous CUDA uint8 tensor")
    if workspace.numel() < need:
        raise ValueError(f"workspace too small: {workspace.numel()} < {need}")


def linear_fp16_pid_ws_out(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, pid: int,
                           workspace: Optional[torch.Tensor], split_k_slices: int = 2) -> None:
    _linear_checks(x, w)
    if x.dtype != torch.float16:
        raise ValueError("input must be fp16")
    S = 2 if split_k_slices <= 0 else split_k_slices
    M, K = x.shape
    N = w.shape[0]
    need = workspace_size(MP_FP16, pid, N, M, K, S)
    _check_workspace(workspace, need)
    ws_bytes = 0 if workspace is None else workspace.numel()
    _check(lib().mp_gemm_rcc_pid(MP_FP16, pid, S, N, M, K, _ptr(w), _ptr(x), _ptr(out), 1.0, 0.0,
                                 _ptr(workspace if need else None), ws_bytes if need else 0, _stream(x)))


def linear_fp16_pid_ws(x: torch.Tensor, w: torch.Tensor, pid: int, workspace: Optional[torch.Tensor],
                       split_k_slices: int = 2) -> torch.Tensor:
    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float16, device=x.device)
    linear_fp16_pid_ws_out(x, w, out, pid, workspace, split_k_slices)
    return out


def fp16_rcc_pid_ws_out(a: torch.Tensor, b_col: torch.Tensor, c_col: torch.Tensor, pid: int,
                        workspace: Optional[torch.Tensor], split_k_slices: int = 2) -> None:
    """a [m,k] row-major; b_col [k,n] with strides (1,k); c_col [m,n] with strides (1,m)
    (moonpoly/core/moonpoly_gemm.cu:438-443)."""
    m, k = a.shape
    n = b_col.shape[1]
    if b_col.stride() != (1, k) or c_col.stride() != (1, m):
        raise ValueError("b_col / c_col must be column-major")
    S = 2 if split_k_slices <= 0 else split_k_slices
    need = workspace_size(MP_FP16, pid, m, n, k, S)
    _check_workspace(workspace, need)
    ws_bytes = 0 if workspace is None else workspace.numel()
    _check(lib().mp_gemm_rcc_pid(MP_FP16, pid, S, m, n, k, _ptr(a), _ptr(b_col), _ptr(c_col), 1.0, 0.0,
                                 _ptr(workspace if need else None), ws_bytes if need else 0, _stream(a)))


def linear_cpp_forced_pid(x: torch.Tensor, w: torch.Tensor, pid: int, split_k: int) -> torch.Tensor:
    """moonpoly.linear_cpp_forced_pid (moonpoly/core/moonpoly_gemm.cu:237-286): non-fp16, non-2-D or
    non-contiguous inputs fall back to `linear`; otherwise the forced pid with run-time split-K."""
    if (x.dtype != torch.float16 or w.dtype != torch.float16 or x.dim() != 2 or w.dim() != 2
            or not x.is_contiguous() or not w.is_contiguous()):
        return linear(x, w)
    S = 2 if split_k <= 0 else split_k
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.float16, device=x.device)
    # no caller workspace here: the library uses its own per-stream scratch
    _check(lib().mp_gemm_rcc_pid(MP_FP16, pid, S, N, M, K, _ptr(w), _ptr(x), _ptr(out), 1.0, 0.0,
                                 ctypes.c_void_p(0), 0, _stream(x)))
    return out


def scaled_int8_mm(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
                   bias: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """moonpoly.scaled_int8_mm (moonpoly/core/moonpoly_gemm.cu:1738-1782): a [M,K] int8, b [K,N] int8
    (pass `weight.t()` for a copy-free call), per-tensor or per-token / per-channel fp32 scales,
    optional bias of the output type; returns [M,N] in `out_dtype` (fp16 or bf16)."""
    if a.dtype != torch.int8 or b.dtype != torch.int8:
        raise ValueError("A and B must be int8")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError("A must be [M,K] and B [K,N]")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("Unsupported output dtype")
    M, K = a.shape
    N = b.shape[1]
    a = a.contiguous()
    b_nk = b.t().contiguous()          # no copy when the caller passed weight.t()
    a_scales = a_scales.to(torch.float32).contiguous().reshape(-1)
    b_scales = b_scales.to(torch.float32).contiguous().reshape(-1)
    if a_scales.numel() not in (1, M) or b_scales.numel() not in (1, N):
        raise ValueError("scales must be scalars or per-token [M,1] / per-channel [1,N]")
    if bias is not None:
        if bias.dtype != out_dtype:
            raise ValueError("Bias dtype mismatch")
        bias = bias.contiguous().reshape(-1)
        if bias.numel() != N:
            raise ValueError("bias must have N elements")
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _check(lib().mp_scaled_mm_i8(M, N, K, _ptr(a), K, _ptr(b_nk), K, _ptr(a_scales), int(a_scales.numel() == 1),
                                 _ptr(b_scales), int(b_scales.numel() == 1), _ptr(bias), _ptr(out), N,
                                 0 if out_dtype == torch.float16 else 1, _stream(a)))
    return out


# ------------------------------------------------------------------------------------------------
# fused all-gather Linear: peer-mapped output buffers and the flag barrier (see shard.PeerOutput)
# ------------------------------------------------------------------------------------------------
def peer_alloc(nbytes: int):
    """(device pointer, 64-byte IPC handle) of a zero-filled buffer other processes of the box can map."""
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    _check(lib().mp_peer_alloc(nbytes, ctypes.byref(ptr), handle))
    return ptr.value, handle.raw


def peer_open(handle: bytes) -> int:
    ptr = ctypes.c_void_p()
    _check(lib().mp_peer_open(handle, ctypes.byref(ptr)))
    return ptr.value


def peer_close(ptr: int) -> None:
    _check(lib().mp_peer_close(ctypes.c_void_p(ptr)))


def peer_free(ptr: int) -> None:
    _check(lib().mp_peer_free(ctypes.c_void_p(ptr)))


def linear_gather(x: torch.Tensor, w_shard: torch.Tensor, dst_ptrs, ld_dst: int, col_offset: int) -> None:
    """mp_linear_gather: Y[:, col_offset : col_offset + N_local] = X @ W_shard^T stored into every buffer of
    `dst_ptrs` (device pointers of the full row-major output [M, ld_dst], this GPU's first)."""
    _linear_checks(x, w_shard)
    M, K = x.shape
    n_local = w_shard.shape[0]
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[ctypes.c_void_p(int(p)) for p in dst_ptrs])
    _check(lib().mp_linear_gather(_dtype_code(x), M, n_local, K, _ptr(x), _ptr(w_shard), arr, len(dst_ptrs), ld_dst,
                                  col_offset, _stream(x)))


def peer_barrier(flag_table: torch.Tensor, world: int, rank: int, value: int, timeout_us: int = 0) -> None:
    """mp_peer_barrier on the current stream; flag_table is a device int64 tensor of `world` flag-array pointers."""
    _check(lib().mp_peer_barrier(_ptr(flag_table), world, rank, value, timeout_us, _stream(flag_table)))


# ------------------------------------------------------------------------------------------------
# timing helper used by the refit and the benchmark
# ------------------------------------------------------------------------------------------------
def time_rcc_pid(dtype: int, pid: int, split_k: int, m: int, n: int, k: int, in_dtype, out_dtype,
                 warmup: int = 5, iters: int = 20, pool_bytes: int = 512 << 20) -> float:
    """Average milliseconds of one forced-pid launch, CUDA events around `iters` back-to-back
    launches that rotate through enough operand copies to exceed L2."""
    dev = torch.device("cuda")
    per = (m * k + n * k) * torch.empty((), dtype=in_dtype).element_size()
    copies = max(1, min(16, pool_bytes // max(per, 1)))
    if in_dtype == torch.int8:
        As = [torch.randint(-3, 3, (m, k), dtype=torch.int8, device=dev) for _ in range(copies)]
        Bs = [torch.randint(-3, 3, (n, k), dtype=torch.int8, device=dev) for _ in range(copies)]
    else:
        As = [torch.randn((m, k), dtype=in_dtype, device=dev) * 0.05 for _ in range(copies)]
        Bs = [torch.randn((n, k), dtype=in_dtype, device=dev) * 0.05 for _ in range(copies)]
    c = torch.empty((n, m), dtype=out_dtype, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    L = lib()

    def call(i):
        _check(L.mp_gemm_rcc_pid(dtype, pid, split_k, m, n, k, _ptr(As[i % copies]), _ptr(Bs[i % copies]),
                                 _ptr(c), 1.0, 0.0, ctypes.c_void_p(0), 0, st))

    for i in range(warmup):
        call(i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(iters):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters
