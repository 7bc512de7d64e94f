"""Host side of bench.py: the reference arm's JSON line (the CPU oracle timed on the sweep's shapes), the pieces of the
workload description both arms share, and that ranks other than 0 stay silent in the reference arm.  No GPU needed."""
import json
import os
import subprocess
import sys

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _run(args, env_extra=None):
    env = dict(os.environ, **(env_extra or {}))
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True, text=True, env=env,
                          timeout=900, cwd=ROOT)


def test_reference_arm_prints_the_contract_line():
    out = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 0 and line["ms_per_step"] > 0
    assert line["higher_is_better"] is True and line["scaling"] == "weak" and line["vs_baseline"] is None
    assert line["dtype"] == "f16" and line["data"] == "synthetic"
    cfg = line["config"]
    assert cfg["workload"].startswith("fp16_rcc_dynamic_m_sweep") and cfg["n"] == 4096 and cfg["k"] == 4096
    assert cfg["sweep_m"] == [1, 2, 4, 8, 16, 32, 64, 127, 128, 255, 512, 1023, 2048, 4096]
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and cpu["sample"]
    assert set(cpu["per_shape_tflops"]) == {str(m) for m in cfg["sweep_m"]}
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_other_ranks_print_nothing():
    out = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
               {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29599"})
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip() == ""


def test_workload_description_is_shared_by_both_arms():
    sys.path.insert(0, ROOT)
    import bench
    cfg = bench.sweep_config(1)
    assert sum(cfg["reps_per_shape"].values()) == 184 and cfg["launch"].startswith("per shape")
    assert bench.sweep_config(8, "stream")["parallelism"].startswith("column-parallel x8")
    assert sum(bench.reps_for(m) for m in bench.SWEEP_M) % bench.WEIGHT_COPIES == 0     # weight copies rotate evenly
    assert bench.WEIGHT_COPIES * 2 * bench.N_DIM * bench.K_DIM > 126 << 20              # more than L2
    assert bench.flops(4096) == 2.0 * 4096 ** 3
    assert bench.algo_bytes(1) == 2.0 * (4096 + 4096 * 4096 + 4096)
    assert abs(bench.geomean([1.0, 4.0]) - 2.0) < 1e-12
