"""The unquantized-Linear path a serving engine runs on top of the `moonpoly_ops` operators.

This is the consumer side of the reference's vLLM integration (integrations/vllm/v0.10.0/
moonpoly_linear.patch: `_apply_moonpoly_linear`, :645-712, and the branches it tries, :487-643),
written for this library: the same environment switches with the same names and defaults, the same
order of attempts, the same operator calls.  A layer's forward goes through, in order,

  1. the C++ selector op   `moonpoly_ops.linear_cpp_selector`      (VLLM_USE_MOONPOLY_CPP_SELECTOR=1)
  2. the pid whitelist     `fp16_workspace_size` + `linear_fp16_pid_ws_out` with the (pid, split_k) a
                           decode-selector table names for (M, N, K)  (VLLM_USE_MOONPOLY_PID_WHITELIST=1)
  3. the split-K / stream-K pid with a pooled workspace for decode shapes
                           (VLLM_USE_MOONPOLY_STREAMK, default on; pid VLLM_MOONPOLY_STREAMK_PID, default 40)
  4. `moonpoly_ops.linear` (with a bias: `moonpoly_ops.linear_bias`, which adds it inside the GEMM's epilogue with
     the same result; VLLM_MOONPOLY_FUSE_BIAS=0 keeps the separate add)

and every attempt that raises or produces a non-finite value falls through to the next one; `None`
tells the caller to use its own GEMM.  Inputs of any rank are flattened to 2-D and the output is
viewed back; a bias is added after the GEMM in the output type.  Workspaces come from a pool keyed
by (device, stream) that only grows.  Nothing here computes: every product is an operator call.

The decode-selector table of the reference is tuned for another GPU, so the table here starts empty
(the library's C++ selector holds the measured plans of this GPU); `load_decode_selector` fills it
from a mapping, `decode_selector_from_patch` reads the reference's table out of its patch file.

`install(module)` swaps the `apply` of a serving engine's UnquantizedLinearMethod for `apply` below,
keeping the original as the fall-back -- what applying the reference's patch does to vLLM 0.10.
"""
from __future__ import annotations

import os
import re
import threading
from typing import Callable, Dict, Optional, Tuple

import torch

_LOCK = threading.Lock()
_WS_POOL: Dict[Tuple[int, int], torch.Tensor] = {}
DECODE_SELECTOR: Dict[Tuple[int, int, int], Tuple[int, int]] = {}
STATS = {"cpp_selector": 0, "whitelist_attempt": 0, "whitelist_hit": 0, "whitelist_fallback": 0,
         "whitelist_unmapped": 0, "streamk_attempt": 0, "streamk_success": 0, "streamk_fallback": 0,
         "streamk_skipped": 0, "linear": 0, "declined": 0}


def _flag(name: str, default: str) -> bool:
    return os.getenv(name, default) == "1"


def _int_set(name: str) -> set:
    return {int(t) for t in os.getenv(name, "").split(",") if t.strip()}


def _ops():
    """The operator namespace; None when the extension has not been imported."""
    ns = getattr(torch.ops, "moonpoly_ops", None)
    return ns if ns is not None and hasattr(ns, "linear") else None


def reset_stats() -> None:
    for k in STATS:
        STATS[k] = 0


def load_decode_selector(table: Dict[Tuple[int, int, int], Tuple[int, int]]) -> None:
    """(M, N, K) -> (pid, split_k) entries for the pid-whitelist branch (replaces the current table)."""
    DECODE_SELECTOR.clear()
    DECODE_SELECTOR.update({tuple(int(v) for v in k): (int(p), int(s)) for k, (p, s) in table.items()})


def decode_selector_from_patch(path: str) -> Dict[Tuple[int, int, int], Tuple[int, int]]:
    """Reads the `(m, n, k): (pid, split_k)` rows of the reference's patch file (its merged decode selector)."""
    rows = {}
    with open(path) as fh:
        for m in re.finditer(r"^\+\s*\((\d+),\s*(\d+),\s*(\d+)\):\s*\((\d+),\s*(\d+)\),", fh.read(), flags=re.M):
            rows[(int(m.group(1)), int(m.group(2)), int(m.group(3)))] = (int(m.group(4)), int(m.group(5)))
    return rows


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A uint8 buffer of at least `nbytes` for (device, current stream); the pool only grows."""
    need = max(int(nbytes), 1)
    key = (int(device.index or 0), int(torch.cuda.current_stream(device).cuda_stream))
    with _LOCK:
        buf = _WS_POOL.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.empty((need,), device=device, dtype=torch.uint8)
            _WS_POOL[key] = buf
        return buf


def streamk_shape_allowed(m: int, n: int, k: int) -> bool:
    """Decode-like shapes only: few tokens, both weight extents large; narrowed further by the
    VLLM_MOONPOLY_STREAMK_MAX_M / _ALLOW_M / _ALLOW_N / _ALLOW_K switches."""
    if m >= 16 or n < 5120 or k < 5120:
        return False
    max_m = int(os.getenv("VLLM_MOONPOLY_STREAMK_MAX_M", "16"))
    if max_m > 0 and m > max_m:
        return False
    for name, v in (("VLLM_MOONPOLY_STREAMK_ALLOW_M", m), ("VLLM_MOONPOLY_STREAMK_ALLOW_N", n),
                    ("VLLM_MOONPOLY_STREAMK_ALLOW_K", k)):
        allowed = _int_set(name)
        if allowed and v not in allowed:
            return False
    return True


def _forced_pid(ops, x2: torch.Tensor, w: torch.Tensor, pid: int, split_k: int) -> torch.Tensor:
    """fp16_workspace_size -> pooled workspace -> linear_fp16_pid_ws_out, then the finiteness check of the
    reference's branches."""
    nbytes = int(ops.fp16_workspace_size(x2, w, pid, split_k))
    ws = workspace(x2.device, nbytes)
    if nbytes > 0:
        ws.zero_()
    out = torch.empty((x2.shape[0], w.shape[0]), device=x2.device, dtype=x2.dtype)
    ops.linear_fp16_pid_ws_out(x2, w, out, pid, ws, split_k)
    if not torch.compiler.is_compiling() and not torch.isfinite(out).all():
        raise RuntimeError(f"non-finite output (pid={pid}, split_k={split_k})")
    return out


def apply_moonpoly_linear(weight: torch.Tensor, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x[..., K] @ weight[N, K]^T (+ bias) through the operators, or None when this path declines (switch off, not
    CUDA, not fp16, operators missing): the caller then runs its own GEMM."""
    if not _flag("VLLM_USE_MOONPOLY_LINEAR", "0"):
        return None
    ops = _ops()
    if (ops is None or x.device.type != "cuda" or weight.device.type != "cuda" or x.dtype != torch.float16
            or weight.dtype != torch.float16 or x.shape[-1] != weight.shape[1]):
        STATS["declined"] += 1
        return None
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    w = weight.contiguous()
    m, n, k = int(x2.shape[0]), int(w.shape[0]), int(x2.shape[1])
    out = None

    if _flag("VLLM_USE_MOONPOLY_CPP_SELECTOR", "0") and hasattr(ops, "linear_cpp_selector"):
        try:
            out = ops.linear_cpp_selector(x2, w)
            STATS["cpp_selector"] += 1
        except Exception:
            out = None
    if out is None and _flag("VLLM_USE_MOONPOLY_PID_WHITELIST", "0"):
        choice = DECODE_SELECTOR.get((m, n, k))
        if choice is None:
            STATS["whitelist_unmapped"] += 1
        else:
            STATS["whitelist_attempt"] += 1
            try:
                out = _forced_pid(ops, x2, w, choice[0], choice[1])
                STATS["whitelist_hit"] += 1
            except Exception:
                STATS["whitelist_fallback"] += 1
                out = None
    if out is None and _flag("VLLM_USE_MOONPOLY_STREAMK", "1"):
        if streamk_shape_allowed(m, n, k):
            STATS["streamk_attempt"] += 1
            try:
                out = _forced_pid(ops, x2, w, int(os.getenv("VLLM_MOONPOLY_STREAMK_PID", "40")),
                                  int(os.getenv("VLLM_MOONPOLY_STREAMK_SPLITK", "2")))
                STATS["streamk_success"] += 1
            except Exception:
                STATS["streamk_fallback"] += 1
                out = None
        else:
            STATS["streamk_skipped"] += 1
    if out is None:
        try:
            if bias is not None and _flag("VLLM_MOONPOLY_FUSE_BIAS", "1") and hasattr(ops, "linear_bias") \
                    and bias.dtype == x2.dtype and bias.numel() == n:
                # not in the reference: the bias add rides in the GEMM's epilogue (bit-identical to the separate add)
                out = ops.linear_bias(x2, w, bias)
                bias = None
            else:
                out = ops.linear(x2, w)
            STATS["linear"] += 1
        except Exception:
            STATS["declined"] += 1
            return None
    if bias is not None:
        out = out + bias
    return out.view(*lead, n)


def apply(layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None,
          fallback: Optional[Callable] = None) -> torch.Tensor:
    """Drop-in body of UnquantizedLinearMethod.apply(layer, x, bias): the operators first, `fallback(layer, x, bias)`
    (default torch.nn.functional.linear on the layer's weight) when they decline."""
    out = apply_moonpoly_linear(layer.weight, x, bias)
    if out is not None:
        return out
    if fallback is not None:
        return fallback(layer, x, bias)
    return torch.nn.functional.linear(x, layer.weight, bias)


def install(linear_module=None) -> bool:
    """Routes `UnquantizedLinearMethod.apply` of a serving engine's linear module (default: vllm's
    model_executor.layers.linear) through `apply`, keeping the original method as the fall-back.  Returns False
    when the module cannot be imported."""
    if linear_module is None:
        try:
            import vllm.model_executor.layers.linear as linear_module      # noqa: PLC0415
        except Exception:
            return False
    cls = getattr(linear_module, "UnquantizedLinearMethod", None)
    if cls is None:
        return False
    if getattr(cls.apply, "_moonpoly_installed", False):
        return True
    original = cls.apply

    def patched(self, layer, x, bias=None):
        return apply(layer, x, bias, fallback=lambda la, xx, bb: original(self, la, xx, bb))
    patched._moonpoly_installed = True
    cls.apply = patched
    return True
