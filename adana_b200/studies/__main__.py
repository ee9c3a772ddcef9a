"""Command line of the studies.

    python -m adana_b200.studies sizes --rule Enoki_Scaled --sizes 8 12 16 24 36 [--formula 6N2]
    python -m adana_b200.studies lr-law     <runs root> --opt adamw --omega 4 [--top-k 5] [--bootstrap 200] [--json J] [--svg S]
    python -m adana_b200.studies curvature  <runs root> --opt adamw --omega 4 [--json J] [--svg S]
    python -m adana_b200.studies loss-laws  <runs root> --opts adamw dana-star-mk4 [--form broken] [--formula 6N2] [--baseline adamw] [--svg S]
    python -m adana_b200.studies gpu-hours  <runs root> [--opt O] [--rule R] [--csv C]
    python -m adana_b200.studies size-curves <runs root> --opt O [--svg S]
    python -m adana_b200.studies opt-stats  <experiment dir> [--svg-prefix P]
    python -m adana_b200.studies tau        <tau_stats dir> [--raw] [--all-kinds] [--svg-prefix P]
    python -m adana_b200.studies kappa      <runs root> --n-head H [--svg-prefix P]
    python -m adana_b200.studies savings    <runs root> --opt dana-star-mk4 [--baseline adamw] [--window 1 30] [--json J] [--svg S]
    python -m adana_b200.studies gamma3     <runs root> --opt dana-star-mk4 [--top-k 3] [--kind power] [--json J] [--svg S]
    python -m adana_b200.studies hoyer      <runs root> [--heads 6 8] [--opts adamw dana-star-mk4] [--json J] [--svg S]
    python -m adana_b200.studies sensitivity --bootstrap B1.json B2.json --names adamw dana-mk4 --curvature C.json \
                                            --law 2.5 0.5 0.12 --losses 3.45 3.40 --target-size 36 [--json J]

`<runs root>` is a folder that holds experiment directories (any depth); `--wandb entity/project` reads a W&B project
instead, and `--cache DIR` keeps what was read on disk (`--refresh` to read again).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np

from . import curvature, gamma3, loss_laws, lr_law, panels, savings, sweeps, tau_cdf
from .runs import CachedRuns, LocalRuns, WandbRuns, lr_sweep_table
from .sizes import model_size, size_key


def _source(a):
    if a.wandb:
        entity, project = a.wandb.split("/", 1)
        src = WandbRuns(entity, project)
    else:
        src = LocalRuns(a.root)
    return CachedRuns(src, a.cache, a.refresh) if a.cache else src


def _dump(obj, path):
    def plain(o):
        if isinstance(o, np.ndarray):
            return o.tolist()
        if isinstance(o, (np.floating, np.integer)):
            return o.item()
        raise TypeError(type(o))

    text = json.dumps(obj, indent=1, default=plain)
    if path:
        Path(path).write_text(text)
    else:
        print(text)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m adana_b200.studies", description=__doc__,
                                formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = p.add_subparsers(dest="cmd", required=True)

    def runs_cmd(name):
        s = sub.add_parser(name)
        s.add_argument("root", nargs="?", default=".")
        s.add_argument("--wandb", default=None)
        s.add_argument("--cache", default=None)
        s.add_argument("--refresh", action="store_true")
        s.add_argument("--group", default=None)
        s.add_argument("--rule", default="Enoki_Scaled")
        s.add_argument("--opt", default=None)
        s.add_argument("--omega", type=float, default=None)
        s.add_argument("--omega-tol", type=float, default=0.1)
        s.add_argument("--kappa", type=float, default=None)
        s.add_argument("--lr-coupled-omega", action="store_true")
        s.add_argument("--json", default=None)
        s.add_argument("--svg", default=None)
        return s

    s = sub.add_parser("sizes")
    s.add_argument("--rule", default="Enoki_Scaled")
    s.add_argument("--sizes", type=int, nargs="+", required=True)
    s.add_argument("--formula", default="default")
    s = runs_cmd("lr-law")
    s.add_argument("--top-k", type=int, default=5)
    s.add_argument("--bootstrap", type=int, default=0)
    s.add_argument("--extrapolate", type=int, nargs="*", default=[])
    runs_cmd("curvature")
    s = runs_cmd("loss-laws")
    s.add_argument("--opts", nargs="+", required=True)
    s.add_argument("--form", default="broken", choices=["single", "broken"])
    s.add_argument("--formula", default="default")
    s.add_argument("--baseline", default=None)
    s.add_argument("--compute-weight", action="store_true")
    s = runs_cmd("gpu-hours")
    s.add_argument("--csv", default=None)
    runs_cmd("size-curves")
    s = runs_cmd("kappa")
    s.add_argument("--n-head", type=int, required=True)
    s.add_argument("--kappa-min", type=float, default=0.0)
    s.add_argument("--svg-prefix", default=None)
    s = runs_cmd("savings")
    s.add_argument("--baseline", default="adamw")
    s.add_argument("--window", type=float, nargs=2, default=[1.0, 30.0])
    s = runs_cmd("gamma3")
    s.add_argument("--top-k", type=int, default=5)
    s.add_argument("--kind", default="power", choices=["power", "linear", "exponential"])
    s.add_argument("--fac-min", type=float, default=0.0)
    s.add_argument("--fac-max", type=float, default=float("inf"))
    s = runs_cmd("hoyer")
    s.add_argument("--heads", type=int, nargs="*", default=None)
    s.add_argument("--opts", nargs="*", default=None)
    s = sub.add_parser("sensitivity")
    s.add_argument("--bootstrap", nargs="+", required=True)
    s.add_argument("--names", nargs="+", required=True)
    s.add_argument("--curvature", required=True)
    s.add_argument("--baseline", default=None)
    s.add_argument("--law", type=float, nargs=3, required=True, metavar=("a", "b", "c"))
    s.add_argument("--losses", type=float, nargs="+", required=True)
    s.add_argument("--target-size", type=int, required=True)
    s.add_argument("--rule", default="Enoki_Scaled")
    s.add_argument("--json", default=None)
    s = sub.add_parser("opt-stats")
    s.add_argument("exp_dir")
    s.add_argument("--svg-prefix", default=None)
    s = sub.add_parser("tau")
    s.add_argument("tau_stats_dir")
    s.add_argument("--raw", action="store_true")
    s.add_argument("--all-kinds", action="store_true")
    s.add_argument("--svg-prefix", default=None)
    a = p.parse_args(argv)

    if a.cmd == "sizes":
        for n in a.sizes:
            m = model_size(n, a.rule)
            print(f"{a.rule} {n}: layers {m.n_layer} heads {m.n_head} width {m.n_embd} non_emb {m.non_emb:,} total "
                  f"{m.total_params:,} compute {m.compute_pfh(a.formula):.4g} PFH ({a.formula}) "
                  f"Chinchilla iterations {m.chinchilla_iterations():,}")
        return 0
    if a.cmd == "opt-stats":
        run = LocalRuns(Path(a.exp_dir).parent).fetch()
        run = next(r for r in run if r.id == Path(a.exp_dir).name)
        stats = sweeps.optimizer_statistics(run)
        for k, d in stats.items():
            print(f"{k}: {len(d['value'])} records, last {d['value'][-1]:.4g}" + (f", theory {d['theory'][-1]:.4g}" if "theory" in d else ""))
            if a.svg_prefix:
                panels.optimizer_stats(stats, k, f"{a.svg_prefix}_{k.split('/')[-1]}.svg")
        return 0
    if a.cmd == "tau":
        rep = (tau_cdf.all_kinds if a.all_kinds else tau_cdf.summary)(a.tau_stats_dir, raw=a.raw)
        for name, g in rep["groups"].items():
            last = g["lines"][-1]
            med = float(np.interp(0.5, last["prob"], last["tau"])) if len(last["tau"]) else float("nan")
            print(f"{name}: {g['tensors']} tensors, median at iteration {last['iteration']}: {med:.4g}")
            if a.svg_prefix:
                panels.tau_cdf(g, f"{a.svg_prefix}_{name.replace(' ', '_').replace('.', '_')}.svg", name, a.raw)
        return 0

    if a.cmd == "sensitivity":
        boots = {n: json.loads(Path(f).read_text()) for n, f in zip(a.names, a.bootstrap)}
        boots = {n: b.get("bootstrap", b) for n, b in boots.items()}          # a whole lr-law report or its bootstrap part
        rep = savings.sensitivity(boots, json.loads(Path(a.curvature).read_text()), dict(zip(a.names, a.losses)),
                                  a.baseline or a.names[0], model_size(a.target_size, a.rule).non_emb, *a.law)
        _dump(rep, a.json)
        return 0
    runs = _source(a).fetch({"group": a.group} if a.group else None)
    sel = dict(omega=a.omega, omega_tol=a.omega_tol, kappa=a.kappa, lr_coupled=a.lr_coupled_omega)
    if a.cmd in ("lr-law", "curvature"):
        table = lr_sweep_table(runs, size_key(a.rule), opt=a.opt, **sel)
        if a.cmd == "lr-law":
            rep = lr_law.study(table, a.rule, a.top_k, None, a.bootstrap, extrapolate_sizes=a.extrapolate)
            rep["metadata"]["target_omega"] = a.omega
            if a.svg:
                panels.lr_law(rep, a.svg)
        else:
            rep = curvature.study(table, a.rule)
            if a.svg:
                panels.curvature(rep, table, a.svg)
        _dump(rep, a.json)
        return 0
    if a.cmd == "loss-laws":
        curves = []
        for opt in a.opts:
            best = sweeps.best_runs_per_size(runs, a.rule, opt, **sel)
            if best:
                curves.append({"name": opt, "compute": [model_size(sz, a.rule).compute_pfh(a.formula) for sz in best],
                               "loss": [d["final_loss"] for d in best.values()]})
        fit = loss_laws.fit_joint(curves, a.form, compute_weight=a.compute_weight)
        if a.baseline:
            base = next(c for c in curves if c["name"] == a.baseline)
            fit["multiplier"] = {c["name"]: [x.tolist() for x in loss_laws.multiplier_piecewise(c["compute"], c["loss"], base["compute"], base["loss"])]
                                 for c in curves if c["name"] != a.baseline}
        if a.svg:
            panels.loss_laws(curves, fit, a.svg)
        _dump(fit, a.json)
        return 0
    if a.cmd == "savings":
        base = sweeps.best_runs_per_size(runs, a.rule, a.baseline)
        baselines = {sz: {"final_loss": d["final_loss"], "final_compute": d["compute"][-1] if d["compute"] else float("nan"),
                          "model_compute": model_size(sz, a.rule).compute_pfh(), "non_emb": d["non_emb"]} for sz, d in base.items()}
        cands = {}
        for r in sweeps.select(runs, opt=a.opt, **sel):
            sz = r.config.get(size_key(a.rule))
            if sz is None:
                continue
            m = model_size(int(sz), a.rule)
            toks, losses = r.series("val/loss", x="tokens")
            hist = [(6.0 * m.non_emb * t / 3600e15, l) for t, l in zip(toks, losses)]
            if hist:
                cands.setdefault(int(sz), []).append({"history": hist, "final_compute": hist[-1][0], "run_name": r.name})
        rows = savings.saved_per_size(baselines, cands)
        ds = [{"name": a.opt, "x": [r["model_compute"] for r in rows], "y": [r["compute_saved"] for r in rows]}]
        lines = savings.fit_savings_lines(ds, tuple(a.window))
        if a.svg and rows:
            panels.savings(ds, lines, a.svg)
        _dump({"per_size": rows, "lines": lines}, a.json)
        return 0
    if a.cmd == "gamma3":
        rows = [{"size": int(r.config[size_key(a.rule)]), "iterations": int(r.config["iterations"]),
                 "gamma_3_factor": float(r.config["gamma_3_factor"]), "val_loss": float(r.final_val_loss), "run": r.name}
                for r in sweeps.select(runs, opt=a.opt, need=("gamma_3_factor", "iterations", size_key(a.rule)), **sel)
                if r.final_val_loss is not None]
        rep = gamma3.study(rows, a.rule, a.top_k, a.kind, a.fac_min, a.fac_max)
        if a.svg and rep["points"]:
            panels.gamma3(rep, a.svg)
        _dump(rep, a.json)
        return 0
    if a.cmd == "hoyer":
        by = sweeps.hoyer_loss_by_coefficient(sweeps.hoyer_points(runs, a.heads, a.opts))
        if a.svg and by:
            panels.hoyer(by, a.svg)
            curves = sweeps.hoyer_curves(runs, a.heads[0] if a.heads else None, a.opts[0] if a.opts else None)
            if curves:
                panels.hoyer_curves(curves, str(Path(a.svg).with_suffix("")) + "_curves.svg")
        _dump({f"{h}:{o}": pts for (h, o), pts in by.items()}, a.json)
        return 0
    if a.cmd == "gpu-hours":
        rows = sweeps.gpu_hours_by_size(sweeps.gpu_hours_rows(runs, a.rule, a.opt))
        print(sweeps.gpu_hours_table(rows))
        if a.csv:
            sweeps.write_csv(rows, a.csv)
        return 0
    if a.cmd == "size-curves":
        best = sweeps.best_runs_per_size(runs, a.rule, a.opt, **sel)
        for size, d in best.items():
            print(f"{size}: {d['run']} final {d['final_loss']:.4f}")
        if a.svg:
            panels.size_curves(best, a.svg, a.opt or "")
        return 0
    if a.cmd == "kappa":
        sw = sweeps.kappa_sweep(runs, a.n_head)
        base = sweeps.adamw_baseline(runs, a.n_head)
        sl = sweeps.kappa_slices(sw, a.kappa_min)
        _dump({f"{c:g}": d for c, d in sl.items()}, a.json)
        if a.svg_prefix:
            panels.kappa_curves(sw, a.svg_prefix + "_curves.svg", base, a.kappa_min)
            panels.kappa_slice(sl, a.svg_prefix + "_slice.svg", base)
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
