"""TauStatsCollector: collection schedule, order statistics of the Dana-Star tau buffers, files on disk."""
import json
import pickle

import numpy as np
import pytest
import torch

from adana_b200.config import flags
from adana_b200.logging.tau_stats import TauStatsCollector
from adana_b200.optim.logtime import DanaStarMK4


def _optimizer():
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(64, 32)), torch.nn.Parameter(torch.randn(48))]
    opt = DanaStarMK4([{"params": ps, "param_names": ["a.weight", "b.weight"]}], lr=1e-3, delta=8.0, kappa=0.85,
                      clipsnr=2.0, weight_decay=0.0)
    for _ in range(5):
        for p in ps:
            p.grad = torch.randn_like(p) * (torch.rand_like(p) < 0.3)
        opt.step()
    return opt


def _cfg():
    cfg = flags.defaults()
    cfg.iterations, cfg.eval_interval = 4000, 20
    return cfg


def test_collects_at_doubling_eval_counts_and_writes_order_statistics(tmp_path):
    c = TauStatsCollector(tmp_path, _cfg(), ["a.weight", "b.weight"])
    hits = [i for i in range(1, 400) if c.should_collect(i * 20, True)]
    assert hits == [10, 20, 40, 80, 160] and not c.should_collect(123, False)
    c.collect(_optimizer(), 1234)
    files = sorted((tmp_path / "tau_stats").glob("tau_stats_iter_00001234_*.pkl"))
    assert len(files) == 1
    data = pickle.load(open(files[0], "rb"))
    st = data["tau_statistics"]["a.weight"]
    assert st["shape"] == (64, 32) and st["num_elements"] == 2048
    assert np.all(np.diff(st["largest_order_stats"]) <= 0) and np.all(np.diff(st["smallest_order_stats"]) >= 0)
    meta = json.loads((tmp_path / "tau_stats" / "tau_stats_metadata.json").read_text())
    assert meta["collection_schedule"][:3] == [10, 20, 40]


def test_files_equal_those_of_the_reference_collector(ref_src, tmp_path):
    """Same optimizer state, the reference's collector and this one: same schedule, same pickled statistics, same
    sections in the metadata file."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("ref_tau_stats", ref_src / "optim" / "tau_stats_collector.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    opt, out = _optimizer(), {}
    for name, cls in (("ref", ref.TauStatsCollector), ("ours", TauStatsCollector)):
        folder = tmp_path / name
        c = cls(folder, _cfg(), ["a.weight", "b.weight"])
        hits = [i for i in range(1, 400) if c.should_collect(i * 20, True)]
        c.collect(opt, 77)
        data = pickle.load(open(sorted((folder / "tau_stats").glob("tau_stats_iter_*.pkl"))[0], "rb"))
        meta = json.loads((folder / "tau_stats" / "tau_stats_metadata.json").read_text())
        out[name] = (hits, list(c.collection_eval_steps), data, meta)
    (h1, s1, d1, m1), (h2, s2, d2, m2) = out["ref"], out["ours"]
    assert h1 == h2 and s1 == s2 and set(m1) == set(m2)
    assert set(d1["metadata"]) == set(d2["metadata"]) and d1["metadata"]["iteration"] == d2["metadata"]["iteration"] == 77
    assert set(d1["tau_statistics"]) == set(d2["tau_statistics"])
    for pname, want in d1["tau_statistics"].items():
        got = d2["tau_statistics"][pname]
        assert got["shape"] == want["shape"] and got["num_elements"] == want["num_elements"]
        for key in ("largest_order_stats", "smallest_order_stats"):
            assert np.allclose(np.asarray(got[key]), np.asarray(want[key]))
    for section in ("model_params", "optimizer_params", "training_params", "loss_params", "scheduler_params"):
        assert set(m1[section]) == set(m2[section]), section
