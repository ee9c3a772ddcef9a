"""Metrics sink and the analysis helpers built on it."""
import math

import numpy as np

from adana_b200 import analysis as A
from adana_b200.config.scaling import compute_lr
from adana_b200.logging.metrics import MetricsSink, read_metrics, series


def test_sink_round_trip_and_summary(tmp_path):
    import torch

    sink = MetricsSink(tmp_path)
    for it in range(1, 6):
        sink.log({"tokens": it * 1000, "train/loss": 5.0 / it, "iter_dt": 0.5, "lr": torch.tensor(1e-3),
                  "hist": object(), "bad": float("nan")}, step=it)
    sink.log({"tokens": 5000, "final-val/loss": 0.9}, step=5)
    rows = read_metrics(tmp_path)
    assert len(rows) == 6 and "hist" not in rows[0] and "bad" not in rows[0] and rows[0]["iter"] == 1
    xs, ys = series(rows, "train/loss")
    assert xs == [1, 2, 3, 4, 5] and ys[-1] == 1.0
    s = A.summarize_run(tmp_path, non_emb=1e6, world=4)
    assert s["final-val/loss"]["last"] == 0.9
    assert math.isclose(s["gpu_hours"], 0.5 * 5 * 4 / 3600)
    assert math.isclose(s["compute_pfh"], 6 * 1e6 * 5000 / 3600e15)


def test_compute_saved_on_synthetic_power_law_curves():
    c = np.geomspace(1e-3, 1.0, 200)
    base = (c, 2.0 + c ** -0.1)
    fast = (c, 2.0 + (1.5 * c) ** -0.1)            # reaches any loss with 1/1.5 of the compute
    assert abs(A.compute_saved(base, fast) - (1 - 1 / 1.5)) < 5e-3
    assert abs(A.compute_saved(base, base)) < 1e-9
    slow = (c, 2.0 + (0.5 * c) ** -0.1)
    assert math.isnan(A.compute_saved(base, slow))   # never reaches the baseline's final loss


def test_lr_law_fit_recovers_shipped_coefficients():
    sizes = np.array([7e6, 2e7, 6e7, 1.5e8, 4e8, 1e9, 2.3e9])
    a, b, d = 51.47, 1.564e4, -0.7039
    lr = a * (b + sizes) ** d
    fa, fb, fd, err = A.fit_lr_power_law(sizes, lr)
    assert err < 1e-6 and abs(fd - d) < 1e-3 and abs(math.log(fa / a)) < 0.05
    # the law evaluated through the scaling-rule table agrees with itself at a shipped size
    assert compute_lr("enoki", "adamw", 63_705_728 * 36, kappa=0.85, batch_size=64) > 0
    point, samples = A.bootstrap_lr_law(sizes, lr * np.exp(np.random.default_rng(0).normal(0, 0.02, len(sizes))), n_boot=20)
    assert len(samples) > 5 and abs(point[2] - d) < 0.1


def test_figure_scripts_write_svg(tmp_path):
    """The figure scripts draw from files this framework writes (metrics.jsonl, the theory generators' JSON)."""
    import json

    import numpy as np

    from adana_b200 import figures as F
    from adana_b200.theory import generate as G

    exp = tmp_path / "run"
    exp.mkdir()
    rows = [{"iter": i, "tokens": 1000 * i, "val/loss": 5.0 - 0.3 * np.log(i)} for i in range(1, 40)]
    (exp / "metrics.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    a = F.main(["curves", str(exp), "--out", str(tmp_path / "curves.svg")])
    b = F.main(["compute", f"{exp}:1.5e8", "--out", str(tmp_path / "compute.svg")])
    P = np.array([2e7, 6e7, 1.5e8, 4e8, 1e9])
    (tmp_path / "sizes.json").write_text(json.dumps({"P": P.tolist(), "lr": (12.5 * (2.4e4 + P) ** -0.51).tolist()}))
    c = F.main(["lr-law", str(tmp_path / "sizes.json"), "--out", str(tmp_path / "law.svg")])
    G.main(["hummingbird", "--v", "100", "--d", "24", "--m", "4", "--steps", "60", "--kappa_step", "1.0",
            "--out", str(tmp_path / "h.json")])
    d = F.main(["hummingbird", str(tmp_path / "h.json"), "--out", str(tmp_path / "h.svg")])
    G.main(["hummingbird", "--v", "100", "--d", "24", "--m", "4", "--steps", "60", "--kappa_step", "1.0", "--optimizer", "dana-mk4",
            "--out", str(tmp_path / "h2.json")])
    multi = F.main(["hummingbird-multi", str(tmp_path / "h.json"), str(tmp_path / "h2.json"), "--out", str(tmp_path / "hm.svg")]).read_text()
    assert multi.count("<polyline") == 5 and multi.count(">Adam<") == 1 and "DANA-Star-MK4" in multi and "DANA-MK4" in multi
    G.main(["taustats", "--v", "100", "--d", "24", "--m", "8", "--steps", "70", "--out", str(tmp_path / "t.json")])
    e = F.main(["taustats", str(tmp_path / "t.json"), "--out", str(tmp_path / "t.svg")])
    for f in (a, b, c, d, e):
        text = f.read_text()
        assert text.startswith("<svg") and "<polyline" in text and text.rstrip().endswith("</svg>")
    assert "-0.51" in c.read_text()          # the fitted exponent is in the title
    assert "99.9%" in e.read_text() and "50%" in e.read_text()      # tau statistics are drawn as a dual-tail CDF
