"""The operator-level sweep driver: shape lists, artefact columns and the summary on CPU; a short real sweep on the GPU."""
import csv
import json
import os

import pytest

from moonpoly_b200 import operator_sweep as sweep

# the column list of the reference's operator_raw.csv (benchmarks/tools/reproduce_operator_level.py:22-40)
REFERENCE_COLUMNS = ["shape_index", "qid", "category", "backend", "dtype", "m", "n", "k", "flops", "baseline_ms", "moonpoly_ms",
                     "speedup", "cosine_similarity", "correctness_passed", "status", "error", "wall_seconds"]


def test_shape_lists_and_summary(tmp_path):
    assert list(sweep.RAW_FIELDS) == REFERENCE_COLUMNS
    shapes = sweep.synthetic_shapes(120)
    assert len(shapes) == 120 and shapes == sweep.synthetic_shapes(120)                 # seeded
    assert (shapes[0]["m"], shapes[0]["n"], shapes[0]["k"]) == (1, 1, 1)                 # the degenerate shape is in
    assert any(s["k"] % 8 for s in shapes) and any(s["category"] == "DeepBench" for s in shapes)
    assert all(s["flops"] == 2 * s["m"] * s["n"] * s["k"] for s in shapes)
    f = tmp_path / "shapes.csv"
    f.write_text("qid,m,n,k\n0,1,1,1\n7,16,4096,4096\n1300,512,1024,2048\n")
    rows = sweep.read_shapes(str(f))
    assert [r["qid"] for r in rows] == [0, 7, 1300] and rows[2]["category"] == "DeepBench" and rows[1]["shape_index"] == 2
    recs = []
    for s, sp in zip(rows, (2.0, 0.5, None)):
        for dt in sweep.DTYPES:
            recs.append(dict(s, backend="cublas", dtype=dt, speedup=sp, status="pass" if sp else "process_error"))
    summ = sweep.summarize(recs, 3)
    one = summ["cublas:FP16"]
    assert one["records"] == 3 and one["passed"] == 2 and one["process_errors"] == 1
    assert abs(one["speedup_geomean"] - 1.0) < 1e-12 and one["speedup_max"] == 2.0
    assert one["category_correctness"]["DeepBench"] == {"total": 1, "passed": 0}


@pytest.mark.gpu
def test_short_sweep_on_the_gpu(tmp_path):
    shapes = sweep.synthetic_shapes(28)
    records, summary = sweep.run_sweep(shapes, str(tmp_path), log_every=0)
    assert len(records) == 3 * 28
    bad = [r for r in records if r["status"] != "pass"]
    assert not bad, bad[:3]
    assert all(r["cosine_similarity"] >= 0.99 for r in records)
    with open(tmp_path / "operator_raw.csv", newline="") as fh:
        reader = csv.DictReader(fh)
        assert reader.fieldnames == REFERENCE_COLUMNS
        assert sum(1 for _ in reader) == 84
    assert json.load(open(tmp_path / "operator_summary.json"))["cublas:INT8"]["passed"] == 28
    # the per-shape cache: a second run reads result.json instead of launching anything
    from moonpoly_b200 import api
    before = api.launch_count()
    again, _ = sweep.run_sweep(shapes, str(tmp_path), log_every=0)
    assert api.launch_count() == before and again == records
