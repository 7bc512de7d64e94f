"""Host-side pieces of the refit tool: the piecewise fit, the table emitters' layout and the predictor-quality
metrics (definitions of the reference's benchmarks/tools/plot_fp16_predictor_eval.py:64-105,289-355)."""
import math
import os
import re

from moonpoly_b200 import refit


def test_three_segment_fit_recovers_a_piecewise_line():
    def truth(k):
        return 0.004 + 0.0001 * k if k <= 8 else (0.0048 + 0.0003 * (k - 8) if k <= 32 else 0.012 + 0.0005 * (k - 32))
    xs = list(refit.K_ITERS)
    segs = refit.fit_segments(xs, [truth(k) for k in xs])
    assert len(segs) == 3 and [s[0] for s in segs[:2]] == [8, 32] and segs[2][0] >= 10 ** 6
    for k in (2, 6, 12, 24, 48, 100):
        seg = next(s for s in segs if k <= s[0])
        assert abs(seg[1] * k + seg[2] - truth(k)) < 2e-4
    assert len(refit.fit_segments([4, 8], [0.01, 0.02])) == 1        # too few samples: one segment


def test_emitted_tables_keep_the_artefact_layout(tmp_path):
    fits = {"fp16": {3: {"segments": [[8, 1e-4, 4e-3], [32, 3e-4, 2e-3], [10 ** 6, 5e-4, 1e-3]], "red_fixed": 2e-3, "red_tile": 0.0}}}
    out = tmp_path / "t.inc"
    refit.emit_tables(fits, str(out), "unit test")
    text = out.read_text()
    for name in ("kPidValid", "kSegmentCount", "kSegmentMaxKiter", "kSegmentSlope", "kSegmentIntercept",
                 "kFixedMsPerExtraSlice", "kTileMsPerExtraSlice", "kCandidateCount"):
        assert text.count(name) == 3, name                             # once per dtype namespace
    fp16_block = text[text.index("namespace fitted_fp16"):text.index("namespace fitted_int8")]
    assert "kSegmentCount[] = {0,0,0,3,0," in fp16_block and "kPidValid[] = {0,0,0,1,0," in fp16_block
    assert "{8,32,1000000}" in text


def test_predictor_metrics_definitions():
    rows = []
    # shape A: prediction is the measured best; shape B: prediction is third, 20 % slower than the best
    for pid, pred, ms in ((0, 1.0, 10.0), (1, 2.0, 12.0), (2, 3.0, 15.0), (3, 4.0, 30.0)):
        rows.append({"m": 16, "n": 1024, "k": 1024, "pid": pid, "pred_cost": pred, "measured_ms": ms, "predicted_pid": 0})
    for pid, pred, ms in ((0, 1.0, 12.0), (1, 2.0, 10.0), (2, 3.0, 11.0), (3, 4.0, 30.0)):
        rows.append({"m": 256, "n": 4096, "k": 4096, "pid": pid, "pred_cost": pred, "measured_ms": ms, "predicted_pid": 0})
    q = refit.predictor_metrics(rows)
    assert q["shapes"] == 2 and abs(q["lop_mean"] - 0.1) < 1e-12 and abs(q["lop_max"] - 0.2) < 1e-12
    assert q["top1"] == 0.5 and q["top3"] == 1.0 and q["top5"] == 1.0
    assert abs(q["detail"][0]["spearman_rho"] - 1.0) < 1e-12 and abs(q["detail"][0]["kendall_tau"] - 1.0) < 1e-12
    # shape B: true ranks 3,1,2,4 against predicted 1,2,3,4 -> rho = 1 - 6*6/(4*15) = 0.4
    assert abs(q["detail"][1]["spearman_rho"] - 0.4) < 1e-12
    assert q["detail"][1]["pred_true_rank"] == 3 and math.isclose(q["detail"][1]["kendall_tau"], 1.0 / 3.0)


def test_measured_plan_table_is_smooth_along_the_dynamic_dimension():
    """Rows of one layer and mapping, in order of the dynamic dimension: the measured time of a bucket may not exceed
    1.6 x that of the NEXT (larger) bucket -- a row that does carries a noisy measurement."""
    path = os.path.join(os.path.dirname(__file__), "..", "moonpoly-dev_b200", "csrc", "generated", "mp_decode_selector.inc")
    rows = [tuple(float(v) for v in m.groups()) for m in
            re.finditer(r"\{(\d+),(\d+),(\d+),(\d+),(\d+),(\d+),(\d+),(\d+),([0-9.e+-]+)f\}", open(path).read())]
    assert len(rows) > 100
    groups = {}
    for (m_lo, m_hi, n_lo, n_hi, k, cls, pid, split, ms) in rows:
        if m_lo == m_hi and m_lo >= 1000 and (n_lo != n_hi or n_lo < 1000):
            key, dyn = ("linear", m_lo, k, cls), n_lo          # Linear mapping: m is the layer, n the bucket
        else:
            key, dyn = ("direct", n_lo, k, cls), m_lo
        groups.setdefault(key, []).append((dyn, ms))
    bad = []
    for key, seq in groups.items():
        seq.sort()
        for (d0, t0), (d1, t1) in zip(seq, seq[1:]):
            if t0 > 1.6 * t1:
                bad.append((key, d0, t0, d1, t1))
    assert not bad, bad[:5]
