"""Llama-3-70B-shaped FP16 linear stack, N-sharded column-parallel over the GPUs of one box.

80 layers of four Linear projections (hidden 8192): qkv (N=10240, K=8192), o_proj (8192, 8192),
gate_up (57344, 8192), down (8192, 28672).  Rank r of g owns rows [r*N/g, (r+1)*N/g) of every
weight; activations are replicated synthetic inputs of each projection's K.  The outputs of o_proj
and down (the hidden state every rank needs in full) are reassembled with one all-gather each;
qkv and gate_up outputs stay sharded.  A step draws one token count M (70 % decode, M in [1, 256];
30 % prefill, M in [512, 8192]) and runs all 320 GEMMs through `mp_linear` (online selector).

    python -m moonpoly_b200.stack --steps 64                               (1 GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        --master-port 29511 -m moonpoly_b200.stack --steps 64              (2 GPUs)

Rank 0 prints one JSON line: whole-job TFLOP/s (the FLOPs of the full, unsharded stack divided by
the step time, max over ranks), the roofline fraction (sum over GEMMs of max(FLOPs / tensor peak,
bytes / HBM bandwidth) per rank, divided by the measured time) and the share of the all-gathers.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import time

PROJECTIONS = [("qkv", 10240, 8192, False), ("o_proj", 8192, 8192, True),
               ("gate_up", 57344, 8192, False), ("down", 8192, 28672, True)]   # (name, N, K, gather the output)
LAYERS = 80


def draw_tokens(seed: int, steps: int) -> list:
    """Token count per step: with probability 0.7 uniform in [1, 256], else uniform in [512, 8192]."""
    from . import rng
    return [min(8192, m) for m in rng.mixed_batch_sizes(seed, rng.STREAM_SHAPES, steps)]


def load_peaks(root: str) -> dict:
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"tflops": float(d["bf16_tflops_sustained"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured (sustained)"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def run_stack(rank: int, world: int, dev, dist, steps: int = 64, warmup: int = 3, layers: int = LAYERS,
              gather: str = "nccl", resident_frac: float = 0.85, root: str = None):
    """Runs the stack on an initialised process group (dist is None on one GPU) and returns the result line on
    rank 0 (None elsewhere).  gather: "fused" = the GEMM epilogue stores each slab into every GPU's copy of the
    full output through peer-mapped pointers, then one flag-barrier kernel; "nccl" = ncclAllGather after o_proj and
    down; "auto" = fused while the slab a rank pushes to its peers is small (shard.fused_gather_pays), NCCL beyond;
    "none" = GEMMs only."""
    import torch
    from . import api

    L = api.lib()
    vp = ctypes.c_void_p
    stream = torch.cuda.current_stream()
    st = vp(stream.cuda_stream)
    do_gather = gather != "none" and dist is not None

    # resident layers: as many distinct weight sets as fit in `resident_frac` of the free memory (cycled over the layers)
    shard = [(name, n // world, k, g) for (name, n, k, g) in PROJECTIONS]
    per_layer = sum(n * k * 2 for (_, n, k, _) in shard)
    max_m = 8192
    act_bytes = sum(max_m * k * 2 for k in {k for (_, _, k, _) in shard}) + sum(max_m * n * 2 for (_, n, _, _) in shard) + \
        sum(world * max_m * n * 2 for (_, n, _, g) in shard if g)
    free, _ = torch.cuda.mem_get_info(dev)
    resident = max(1, min(layers, int((resident_frac * free - act_bytes) / per_layer)))
    gen = torch.Generator(device=dev)
    gen.manual_seed(4 + 1000 * rank)
    weights = [[torch.empty((n, k), dtype=torch.float16, device=dev).normal_(0.0, 0.02, generator=gen)
                for (_, n, k, _) in shard] for _ in range(resident)]
    x_in = {k: torch.empty((max_m, k), dtype=torch.float16, device=dev).normal_(0.0, 1.0, generator=gen)
            for k in sorted({k for (_, _, k, _) in shard})}
    y_loc = [torch.empty((max_m * n,), dtype=torch.float16, device=dev) for (_, n, _, _) in shard]
    y_all = [torch.empty((world * max_m * n,), dtype=torch.float16, device=dev) if g else None for (_, n, _, g) in shard]

    tokens = draw_tokens(4, warmup + steps)

    fused = {}
    auto = gather == "auto"
    if do_gather and gather in ("fused", "auto"):
        # peer-mapped copies of the two gathered outputs; when any rank cannot map its peers (no peer access between
        # the GPUs, IPC refused) every rank falls back to ncclAllGather together
        from .shard import PeerOutput, fused_gather_pays
        err = ""
        try:
            for j, (_, n, _, g) in enumerate(shard):
                if g:
                    po = PeerOutput(max_m, n * world, rank, world)
                    fused[j] = (po, (vp * world)(*[vp(int(q)) for q in po.dst]), vp(po.flag_table.data_ptr()))
        except Exception as e:       # noqa: BLE001
            err = str(e)[:120]
        ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            for po, _, _ in fused.values():
                po.close()
            fused = {}
            gather = "nccl (peer mapping unavailable" + (": " + err if err else " on another rank") + ")"
    epoch = [0]

    # pointer objects are built once: a step then costs one ctypes call per GEMM (and per barrier), not a dozen
    # Python object constructions on top of it -- with the weights cut 8 ways those were a third of a decode step
    px = {k: vp(t.data_ptr()) for k, t in x_in.items()}
    pw = [[vp(w.data_ptr()) for w in ws] for ws in weights]
    py = [vp(t.data_ptr()) for t in y_loc]
    fp16 = api.MP_FP16
    linear, linear_gather, peer_barrier = L.mp_linear, L.mp_linear_gather, L.mp_peer_barrier

    def step(m: int) -> None:
        for layer in range(layers):
            ws = pw[layer % resident]
            for j, (_, n, k, g) in enumerate(shard):
                if g and j in fused and (not auto or fused_gather_pays(m, n, world)):
                    _, dst, flag_table = fused[j]
                    rc = linear_gather(fp16, m, n, k, px[k], ws[j], dst, world, n * world, rank * n, st)
                    if rc == 0:
                        epoch[0] += 1
                        rc = peer_barrier(flag_table, world, rank, epoch[0], 0, st)
                    if rc:
                        raise RuntimeError(L.mp_last_error_string().decode())
                    continue
                rc = linear(fp16, m, n, k, px[k], ws[j], py[j], st)
                if rc:
                    raise RuntimeError(L.mp_last_error_string().decode())
                if g and do_gather:
                    dist.all_gather_into_tensor(y_all[j][: world * m * n], y_loc[j][: m * n])

    for i in range(warmup):
        step(tokens[i])
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0 = time.perf_counter()
    for i in range(steps):
        evs[i][0].record(stream)
        step(tokens[warmup + i])
        evs[i][1].record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    if dist is not None:
        dist.barrier()
    assert api.device_status() == 0
    ms = torch.tensor([a.elapsed_time(b) for a, b in evs], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.tolist()
    for po, _, _ in fused.values():
        po.close()
    del weights, x_in, y_loc, y_all
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    root = root or os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", ".."))
    peaks = load_peaks(root)
    ms_steps = tokens[warmup:]
    flops_full = [2.0 * m * sum(n * k for (_, n, k, _) in PROJECTIONS) * layers for m in ms_steps]
    roof_ms = []
    for m in ms_steps:
        t = 0.0
        for (_, n, k, _) in shard:
            f = 2.0 * m * n * k
            b = 2.0 * (m * k + n * k + m * n)
            t += max(f / (peaks["tflops"] * 1e12), b / (peaks["hbm_gbs"] * 1e9))
        roof_ms.append(t * layers * 1e3)
    decode = [i for i, m in enumerate(ms_steps) if m <= 256]
    prefill = [i for i, m in enumerate(ms_steps) if m > 256]

    def agg(idx):
        if not idx:
            return None
        return {"steps": len(idx), "ms_per_step": round(sum(ms[i] for i in idx) / len(idx), 3),
                "tflops": round(sum(flops_full[i] for i in idx) / (sum(ms[i] for i in idx) * 1e-3) / 1e12, 1),
                "roofline_frac": round(sum(roof_ms[i] for i in idx) / sum(ms[i] for i in idx), 4)}
    return {"metric": "llama70b_fp16_linear_stack_tflops", "value": sum(flops_full) / (sum(ms) * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": sum(ms) / len(ms), "higher_is_better": True, "scaling": "strong", "dtype": "f16",
            "data": "synthetic", "roofline_frac": sum(roof_ms) / sum(ms), "decode": agg(decode), "prefill": agg(prefill),
            "host_wall_ms_per_step": wall / steps * 1e3, "per_step_tokens_ms": [[int(m), round(t, 3)] for m, t in zip(ms_steps, ms)],
            "config": {"workload": "Llama-3-70B-shaped FP16 linear stack", "layers": layers, "resident_layers": resident,
                       "gather": gather if world > 1 else "none",
                       "parallelism": f"column-parallel x{world}, all-gather after o_proj and down" if do_gather
                       else f"column-parallel x{world}, no collective", "peaks": peaks,
                       "tokens_min_max": [min(ms_steps), max(ms_steps)]}}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nccl", "none"])
    args = ap.parse_args()

    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    line = run_stack(rank, world, dev, dist, args.steps, args.warmup, args.layers, args.gather)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))
    main()
