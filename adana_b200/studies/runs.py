"""The run table behind every study: one record per training run (id, name, config, summary, history), taken either
from experiment directories this framework wrote (`summary.json` + `metrics.jsonl`) or from a Weights & Biases
project, with a disk cache in front of the slow source, and the selections the studies share (optimizer, finished
runs only, renormalised weight decay omega, kappa, size knob).

The reference's figure scripts each talk to `wandb.Api()` themselves and repeat the same filters
(visualization/lr_curvature_analysis.py:162-270, bighead_lr_scaling.py:449-690, gamma3_factor_scaling.py:170-350);
its visualization/wandb_cache.py wraps the API in a JSON cache.  Here the source is an object with one method,
`fetch(filters) -> list of plain dicts`, so the same study runs offline on local experiment folders, and the cache
(`CachedRuns`) works for any source: run metadata under `<cache>/runs/<source key>_<hash of filters>.json`, histories
under `<cache>/history/<run id>.json`, `force_refresh=True` to go back to the source.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Sequence

from ..logging.metrics import read_metrics

DANA_FAMILY = ("dana-star-mk4", "dana", "dana-mk4", "dana-star", "adana", "adamw-decaying-wd", "ademamix-decaying-wd")


def _plain(obj):
    """JSON-safe copy (numpy scalars, tuples, odd objects) of a config or summary."""
    if isinstance(obj, dict):
        return {str(k): _plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_plain(v) for v in obj]
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    if hasattr(obj, "item"):
        try:
            return obj.item()
        except Exception:
            pass
    return str(obj)


def flatten_config(config) -> Dict:
    """W&B stores config entries as {"value": v, "desc": ...} in some exports, and whole configs as JSON strings in
    others; both become a flat {name: value}."""
    if isinstance(config, str):
        try:
            config = json.loads(config)
        except ValueError:
            return {}
    if hasattr(config, "as_dict"):
        config = config.as_dict()
    return {k: (v["value"] if isinstance(v, dict) and "value" in v else v) for k, v in dict(config or {}).items()}


@dataclass
class Run:
    id: str
    name: str
    config: Dict
    summary: Dict
    _history: Optional[List[Dict]] = None
    _load_history: Optional[Callable[[], List[Dict]]] = field(default=None, repr=False)

    def history(self, keys: Optional[Sequence[str]] = None) -> List[Dict]:
        """Logged records in order; with `keys`, only the records that carry all of them."""
        if self._history is None:
            self._history = list(self._load_history()) if self._load_history else []
        if not keys:
            return self._history
        return [r for r in self._history if all(k in r and r[k] is not None for k in keys)]

    def series(self, key: str, x: str = "iter"):
        rows = self.history([x, key])
        return [r[x] for r in rows], [r[key] for r in rows]

    # ---- the quantities the studies read ----------------------------------------------------------------------------
    @property
    def opt(self) -> str:
        return self.config.get("opt", "")

    @property
    def finished(self) -> bool:
        """False only when both the logged and the configured iteration counts are known and the run stopped short."""
        done, want = self.summary.get("iter", 0) or 0, self.config.get("iterations", 0) or 0
        return not (done > 0 and want > 0 and done < want)

    @property
    def final_val_loss(self) -> Optional[float]:
        return self.summary.get("final-val/loss")

    def omega(self, lr_coupled: bool = False) -> float:
        """Renormalised weight decay.  Optimizers whose decay runs on its own time scale (the ADana family and the
        *-decaying-wd ones, Manau with `wd_decaying`) are launched with wd = omega / wd_ts, so omega = wd * wd_ts;
        the coupled ones (AdamW, AdEMAMix, Muon) with wd = omega / (lr * iterations), so omega = wd * lr *
        iterations.  `lr_coupled=True` multiplies the first form by lr: the convention of the archived sweeps the
        reference's figure scripts read (bighead_lr_scaling.py:640-661), whose decay was still tied to the peak lr."""
        c = self.config
        lr = c.get("lr") or 0.0
        own_clock = self.opt in DANA_FAMILY or self.opt.startswith(("dana-", "adana")) or \
            (self.opt == "manau" and c.get("wd_decaying"))
        if own_clock:
            w = (c.get("wd_ts", 1.0) or 1.0) * (c.get("weight_decay", 1.0) or 0.0)
            return w * lr if lr_coupled else w
        return (c.get("weight_decay", 0.1) or 0.0) * lr * (c.get("iterations", 1) or 1)

    def to_json(self, with_history: bool = False) -> Dict:
        d = {"id": self.id, "name": self.name, "config": _plain(self.config), "summary": _plain(self.summary)}
        if with_history:
            d["history"] = _plain(self.history())
        return d


# ---- sources ---------------------------------------------------------------------------------------------------------
class LocalRuns:
    """Experiment directories under `root` (any depth): a run is a folder with `summary.json`; its history is the
    folder's `metrics.jsonl`.  `filters` are equality tests on config entries ({"opt": "adana"}), with "group"
    matched against `wandb_group` as W&B would."""

    def __init__(self, root):
        self.root = Path(root)
        self.key = "local_" + hashlib.md5(str(self.root.resolve()).encode()).hexdigest()[:8]

    def fetch(self, filters: Optional[Dict] = None) -> List[Run]:
        out = []
        for s in sorted(self.root.rglob("summary.json")):
            try:
                doc = json.loads(s.read_text())
            except ValueError:
                continue
            cfg = flatten_config(doc.get("args", {}))
            if not _matches(cfg, filters):
                continue
            summary = {k: v for k, v in doc.items() if k != "args"}
            exp = s.parent
            rows_file = exp / "metrics.jsonl"
            if rows_file.exists():
                for r in reversed(read_metrics(rows_file)):      # last logged value of every metric, as W&B keeps it
                    for k, v in r.items():
                        summary.setdefault(k, v)
            out.append(Run(exp.name, exp.name, cfg, summary,
                           _load_history=(lambda f=rows_file: read_metrics(f) if f.exists() else [])))
        return out


class WandbRuns:
    """Runs of `<entity>/<project>` through the W&B public API (imported on first use)."""

    def __init__(self, entity: str, project: str, api=None):
        self.path, self._api = f"{entity}/{project}", api
        self.key = self.path.replace("/", "_")

    def fetch(self, filters: Optional[Dict] = None) -> List[Run]:
        if self._api is None:
            import wandb

            self._api = wandb.Api()
        out = []
        for r in self._api.runs(self.path, filters=filters or {}):
            summary = r.summary
            summary = dict(summary._json_dict) if hasattr(summary, "_json_dict") else dict(summary)
            out.append(Run(r.id, r.name, flatten_config(r.config), summary,
                           _load_history=(lambda run=r: [dict(row) for row in run.scan_history()])))
        return out


def _matches(cfg: Dict, filters: Optional[Dict]) -> bool:
    for k, want in (filters or {}).items():
        have = cfg.get("wandb_group") if k == "group" else cfg.get(k)
        if have != want:
            return False
    return True


class CachedRuns:
    """Disk cache in front of a source.  `fetch` returns cached metadata when the same (source, filters) was asked
    before; a run's history is read from the source the first time it is needed and kept in its own file."""

    def __init__(self, source, cache_dir="run_cache", force_refresh: bool = False):
        self.source, self.dir, self.force = source, Path(cache_dir), force_refresh
        (self.dir / "runs").mkdir(parents=True, exist_ok=True)
        (self.dir / "history").mkdir(parents=True, exist_ok=True)
        self.hits = self.misses = 0

    def _runs_file(self, filters) -> Path:
        h = hashlib.md5(json.dumps(filters or {}, sort_keys=True, default=str).encode()).hexdigest()[:12]
        group = str((filters or {}).get("group", "all")).replace("/", "_")
        return self.dir / "runs" / f"{self.source.key}_{group}_{h}.json"

    def _history_file(self, run_id: str) -> Path:
        return self.dir / "history" / f"{run_id}.json"

    def _wrap(self, meta: Dict, live: Optional[Run]) -> Run:
        hf = self._history_file(meta["id"])

        def load():
            if hf.exists() and not self.force:
                return json.loads(hf.read_text())
            src = live
            if src is None:      # metadata came from the cache: ask the source again for this one run
                src = next((r for r in self.source.fetch(None) if r.id == meta["id"]), None)
            rows = _plain(src.history()) if src is not None else []
            hf.write_text(json.dumps(rows))
            return rows

        return Run(meta["id"], meta["name"], meta.get("config", {}), meta.get("summary", {}), _load_history=load)

    def fetch(self, filters: Optional[Dict] = None) -> List[Run]:
        f = self._runs_file(filters)
        if f.exists() and not self.force:
            self.hits += 1
            return [self._wrap(m, None) for m in json.loads(f.read_text())]
        self.misses += 1
        live = self.source.fetch(filters)
        f.write_text(json.dumps([r.to_json() for r in live]))
        return [self._wrap(r.to_json(), r) for r in live]


# ---- selections ------------------------------------------------------------------------------------------------------
def select(runs: Iterable[Run], opt: Optional[str] = None, finished: bool = True, omega: Optional[float] = None,
           omega_tol: float = 0.1, kappa: Optional[float] = None, kappa_tol: float = 0.05,
           need: Sequence[str] = ("lr",), where: Optional[Callable[[Run], bool]] = None,
           lr_coupled: bool = False) -> List[Run]:
    out = []
    for r in runs:
        if opt is not None and r.opt != opt:
            continue
        if finished and not r.finished:
            continue
        if any(r.config.get(k) is None for k in need):
            continue
        if kappa is not None and (r.config.get("kappa") is None or abs(r.config["kappa"] - kappa) > kappa_tol):
            continue
        if omega is not None and abs(r.omega(lr_coupled) - omega) > omega_tol:
            continue
        if where is not None and not where(r):
            continue
        out.append(r)
    return out


def lr_sweep_table(runs: Iterable[Run], size_key: str = "n_head", **sel) -> Dict[int, List[Dict]]:
    """size -> [{lr, val_loss, omega, run}] of the finished runs that carry a final validation loss."""
    table: Dict[int, List[Dict]] = {}
    for r in select(runs, **sel):
        size, loss = r.config.get(size_key), r.final_val_loss
        if size is None or loss is None:
            continue
        table.setdefault(int(size), []).append({"lr": float(r.config["lr"]), "val_loss": float(loss),
                                                "omega": r.omega(sel.get("lr_coupled", False)), "run": r.name})
    return table
