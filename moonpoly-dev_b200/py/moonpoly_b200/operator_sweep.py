"""Operator-level sweep: every shape of a shape list, FP16 / FP32 / INT8 row-column-column GEMM through the
library's online selector, timed against the vendor GEMM of the box and checked by cosine similarity.

Counterpart of the reference's benchmarks/tools/reproduce_operator_level.py (:1-484) and of the C++ programme it
drives (benchmarks/cpp/moonpoly_vs_cublas_benchmark.cu:74,131-176): the same protocol (5 warm-up + 20 timed launches
per shape and dtype, CUDA events, inputs uniform in [-1, 1] / int8 in [-127, 127], cosine similarity >= 0.99 as the
correctness bar), the same per-shape result cache (one result.json per shape directory, reused unless --force), and
the same artefacts with the same columns:

    operator_raw.csv       shape_index,qid,category,backend,dtype,m,n,k,flops,baseline_ms,moonpoly_ms,speedup,
                           cosine_similarity,correctness_passed,status,error,wall_seconds
    operator_summary.json  per (backend, dtype): records, passed, incorrect, missing, speed-up mean / geomean /
                           median / min / max, correctness per category

The shape list is a CSV with columns qid,m,n,k (the reference's benchmarks/data/core/gemm_trick.csv has 1433 rows:
LLM projections, irregular and unaligned shapes down to 1x1x1, and the DeepBench set from qid 1299 on).  Without
--shapes a seeded synthetic list with the same make-up is generated.  The baseline ("cublas" in the backend column)
is torch.matmul for FP16 / FP32 and torch._int_mm for INT8 where it accepts the shape: harness only, the library
itself never calls a vendor GEMM.

    python -m moonpoly_b200.operator_sweep --outdir out/operator_level [--shapes gemm_trick.csv] [--limit N]
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import os
import statistics
import sys
import time

RAW_FIELDS = ("shape_index", "qid", "category", "backend", "dtype", "m", "n", "k", "flops", "baseline_ms", "moonpoly_ms",
              "speedup", "cosine_similarity", "correctness_passed", "status", "error", "wall_seconds")
DTYPES = ("FP16", "FP32", "INT8")
WARMUP, ITERS = 5, 20
COSINE_BAR = 0.99


def synthetic_shapes(count: int = 200, seed: int = 7):
    """A seeded stand-in for the reference's shape list: degenerate and tiny shapes, unaligned K, LLM projection
    shapes with small token counts, irregular mid-size shapes, and a DeepBench-like block from qid 1299 on."""
    from . import rng
    shapes = [(1, 1, 1), (1, 1, 3), (2, 2, 2), (2, 2, 4), (3, 5, 7), (17, 33, 65), (64, 64, 64), (127, 129, 131)]
    u = rng.uniform01(seed, 9, 6 * count)
    llm_nk = [(4096, 4096), (6144, 4096), (28672, 4096), (4096, 14336), (5120, 5120), (15360, 5120), (5120, 13824),
              (10240, 8192), (8192, 8192), (1024, 8192)]
    i = 0
    while len(shapes) < count:
        kind = int(u[i] * 4)
        if kind == 0:       # decode / prefill rows against an LLM projection (RCC m = tokens, n = N)
            n, k = llm_nk[int(u[i + 1] * len(llm_nk))]
            m = max(1, int(round(8192 ** u[i + 2])))
            shapes.append((m, n, k))
        elif kind == 1:     # irregular, K not a multiple of 8
            shapes.append((1 + int(u[i + 1] * 700), 1 + int(u[i + 2] * 3000), 1 + int(u[i + 3] * 4000)))
        elif kind == 2:     # aligned mid-size
            shapes.append((8 * (1 + int(u[i + 1] * 256)), 8 * (1 + int(u[i + 2] * 512)), 64 * (1 + int(u[i + 3] * 64))))
        else:               # square-ish powers of two with a ragged edge
            b = 2 ** (5 + int(u[i + 1] * 8))
            shapes.append((b - int(u[i + 2] * 3), b, b + 8 * int(u[i + 3] * 3)))
        i += 6
    rows = []
    for idx, (m, n, k) in enumerate(shapes[:count]):
        qid = idx if idx < count * 9 // 10 else 1299 + idx
        rows.append({"shape_index": idx + 1, "qid": qid, "category": "DeepBench" if qid >= 1299 else "Real-World",
                     "m": m, "n": n, "k": k, "flops": 2 * m * n * k})
    return rows


def read_shapes(path: str):
    rows = []
    with open(path, newline="") as fh:
        reader = csv.DictReader(fh)
        if reader.fieldnames is None or not {"m", "n", "k"}.issubset(reader.fieldnames):
            raise ValueError(f"shape CSV must have m,n,k columns: {path}")
        for i, r in enumerate(reader, start=1):
            qid = int(r.get("qid", r.get("id", i - 1)))
            m, n, k = int(r["m"]), int(r["n"]), int(r["k"])
            rows.append({"shape_index": i, "qid": qid, "category": "DeepBench" if qid >= 1299 else "Real-World",
                         "m": m, "n": n, "k": k, "flops": 2 * m * n * k})
    return rows


def _time_ms(fn):
    import torch
    for _ in range(WARMUP):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(ITERS):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / ITERS


def _cosine(x, y):
    import torch
    x, y = x.double().flatten(), y.double().flatten()
    nx, ny = torch.linalg.vector_norm(x), torch.linalg.vector_norm(y)
    if nx == 0 and ny == 0:
        return 1.0
    if nx == 0 or ny == 0:
        return 0.0
    return float(torch.dot(x, y) / (nx * ny))


def run_shape(shape: dict, seed: int = 0):
    """The three dtypes of one shape: [record per dtype] (RCC: A [m,k] row-major, B stored [n,k], C stored [n,m])."""
    import torch
    from . import api
    m, n, k = shape["m"], shape["n"], shape["k"]
    dev = "cuda"
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + shape["qid"])
    records = []
    t_start = time.perf_counter()
    for dtype in DTYPES:
        rec = dict(shape, backend="cublas", dtype=dtype, baseline_ms=None, moonpoly_ms=None, speedup=None,
                   cosine_similarity=None, correctness_passed=False, status="missing", error="", wall_seconds=None)
        try:
            if dtype == "INT8":
                a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev, generator=gen)
                b = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev, generator=gen)
                ref = (a.double() @ b.double().t()).t()                 # exact: |sum| < 2^53
                base = None
                if m > 16 and k % 8 == 0 and n % 8 == 0:
                    try:
                        bt = b.t()
                        base = lambda: torch._int_mm(a, bt)              # noqa: E731
                        base()
                    except Exception:
                        base = None
            else:
                tdt = torch.float16 if dtype == "FP16" else torch.float32
                a = (torch.rand((m, k), device=dev, generator=gen) * 2 - 1).to(tdt)
                b = (torch.rand((n, k), device=dev, generator=gen) * 2 - 1).to(tdt)
                ref = (a.double() @ b.double().t()).t()
                bt = b.t()
                base = lambda: torch.matmul(a, bt)                       # noqa: E731
            c = torch.empty((n, m), dtype=torch.int32 if dtype == "INT8" else a.dtype, device=dev)
            ours = lambda: api.gemm_rcc(a, b, c_nm=c)                    # noqa: E731
            ours()
            torch.cuda.synchronize()
            cos = _cosine(c, ref)
            rec["moonpoly_ms"] = round(_time_ms(ours), 6)
            if base is not None:
                rec["baseline_ms"] = round(_time_ms(base), 6)
                rec["speedup"] = round(rec["baseline_ms"] / rec["moonpoly_ms"], 6)
            rec["cosine_similarity"] = round(cos, 9)
            rec["correctness_passed"] = bool(cos >= COSINE_BAR and math.isfinite(cos))
            rec["status"] = "pass" if rec["correctness_passed"] else "incorrect"
            if not rec["correctness_passed"]:
                rec["error"] = "Cosine similarity threshold failed"
        except Exception as e:       # one bad shape must not end the sweep
            rec["status"] = "process_error"
            rec["error"] = str(e)[:300]
        records.append(rec)
    wall = time.perf_counter() - t_start
    for rec in records:
        rec["wall_seconds"] = round(wall, 4)
    return records


def _geomean(values):
    vals = [v for v in values if v and v > 0 and math.isfinite(v)]
    return math.exp(sum(math.log(v) for v in vals) / len(vals)) if vals else None


def summarize(records, expected_shapes: int):
    out = {}
    for dtype in DTYPES:
        sel = [r for r in records if r["dtype"] == dtype]
        passed = [r for r in sel if r["status"] == "pass"]
        sp = [float(r["speedup"]) for r in passed if r["speedup"] is not None]
        cats = {}
        for cat in ("Real-World", "DeepBench"):
            rows = [r for r in sel if r["category"] == cat]
            cats[cat] = {"total": len(rows), "passed": sum(r["status"] == "pass" for r in rows)}
        out[f"cublas:{dtype}"] = {
            "expected_shapes": expected_shapes, "records": len(sel), "passed": len(passed),
            "incorrect": sum(r["status"] == "incorrect" for r in sel), "missing": sum(r["status"] == "missing" for r in sel),
            "process_errors": sum(r["status"] == "process_error" for r in sel),
            "with_baseline": len(sp), "speedup_avg": statistics.fmean(sp) if sp else None, "speedup_geomean": _geomean(sp),
            "speedup_median": statistics.median(sp) if sp else None, "speedup_min": min(sp) if sp else None,
            "speedup_max": max(sp) if sp else None, "category_correctness": cats}
    return out


def run_sweep(shapes, outdir: str, force: bool = False, log_every: int = 100):
    """Runs (or reloads from the per-shape cache) every shape; writes operator_raw.csv, operator_summary.json and
    manifest.json under `outdir`; returns (records, summary)."""
    os.makedirs(outdir, exist_ok=True)
    records = []
    for i, shape in enumerate(shapes):
        run_dir = os.path.join(outdir, "runs", f"qid_{shape['qid']:04d}_{shape['m']}x{shape['n']}x{shape['k']}")
        cache = os.path.join(run_dir, "result.json")
        if os.path.exists(cache) and not force:
            with open(cache) as fh:
                recs = json.load(fh)["records"]
        else:
            recs = run_shape(shape)
            os.makedirs(run_dir, exist_ok=True)
            tmp = cache + ".tmp"
            with open(tmp, "w") as fh:
                json.dump({"shape": shape, "records": recs}, fh)
            os.replace(tmp, cache)
        records += recs
        if log_every and (i + 1) % log_every == 0:
            print(f"[operator_sweep] {i + 1}/{len(shapes)} shapes", file=sys.stderr, flush=True)
    with open(os.path.join(outdir, "operator_raw.csv"), "w", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=RAW_FIELDS, extrasaction="ignore")
        w.writeheader()
        w.writerows(records)
    summary = summarize(records, len(shapes))
    with open(os.path.join(outdir, "operator_summary.json"), "w") as fh:
        json.dump(summary, fh, indent=2)
    with open(os.path.join(outdir, "manifest.json"), "w") as fh:
        json.dump({"shapes": len(shapes), "protocol": {"warmup": WARMUP, "iters": ITERS, "cosine_bar": COSINE_BAR},
                   "baseline": "torch.matmul (FP16, FP32), torch._int_mm (INT8 where it accepts the shape)"}, fh, indent=2)
    return records, summary


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default=None, help="CSV with qid,m,n,k; default: a seeded synthetic list")
    ap.add_argument("--outdir", default="out/operator_level")
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--synthetic-count", type=int, default=200, dest="synthetic_count")
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    shapes = read_shapes(args.shapes) if args.shapes else synthetic_shapes(args.synthetic_count)
    if args.limit > 0:
        shapes = shapes[: args.limit]
    _, summary = run_sweep(shapes, args.outdir, args.force)
    print(json.dumps({k: {kk: v[kk] for kk in ("records", "passed", "incorrect", "process_errors", "speedup_avg",
                                                  "speedup_geomean", "speedup_max")} for k, v in summary.items()}))


if __name__ == "__main__":
    sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))
    main()
