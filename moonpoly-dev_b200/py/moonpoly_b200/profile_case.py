"""Run one GEMM shape a few times through the C ABI: the small case that profiler captures use.

    python moonpoly-dev_b200/py/moonpoly_b200/profile_case.py --dtype fp16 --m 4096 --n 4096 --k 4096 --launches 3
    python ... --pid 400 --split-k 4          (forced pid instead of the online selector)
    python ... --dtype int8 --scaled          (INT8 scaled matmul; m = tokens, n = channels)
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

import torch  # noqa: E402

from moonpoly_b200 import api  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "int8", "fp32"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--pid", type=int, default=None)
    ap.add_argument("--split-k", type=int, default=1, dest="split_k")
    ap.add_argument("--scaled", action="store_true")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--copies", type=int, default=2, help="operand copies rotated between launches")
    args = ap.parse_args()
    dev = "cuda"
    tdt = {"fp16": torch.float16, "int8": torch.int8, "fp32": torch.float32}[args.dtype]

    def operand(rows):
        if tdt == torch.int8:
            return torch.randint(-127, 128, (rows, args.k), dtype=torch.int8, device=dev)
        return (torch.randn((rows, args.k), device=dev) * 0.05).to(tdt)

    As = [operand(args.m) for _ in range(args.copies)]
    Bs = [operand(args.n) for _ in range(args.copies)]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.scaled:
        sa = torch.rand((args.m,), device=dev) * 0.019 + 0.001
        sb = torch.rand((args.n,), device=dev) * 0.019 + 0.001
    e0.record()
    for i in range(args.launches):
        a, b = As[i % args.copies], Bs[i % args.copies]
        if args.scaled:
            api.scaled_int8_mm(a, b.t(), sa, sb)
        elif args.pid is None:
            api.gemm_rcc(a, b)
        else:
            api.gemm_rcc_pid(a, b, args.pid, args.split_k)
    e1.record()
    torch.cuda.synchronize()
    assert api.device_status() == 0
    print(f"{args.dtype} m={args.m} n={args.n} k={args.k} pid={args.pid} split_k={args.split_k}: "
          f"{e0.elapsed_time(e1) / args.launches * 1e3:.2f} us per launch over {args.launches} launches")


if __name__ == "__main__":
    main()
