"""Local metrics sink: every scalar the trainer reports also lands in `<exp_dir>/metrics.jsonl`.

The reference reports only to Weights & Biases (src/optim/base.py:302-357; its plotting scripts read the
W&B API).  Here the same records — same metric names (`iter`, `tokens`, `train/loss`, `val/loss`,
`final-val/loss`, `iter_dt`, `lr`, `optimizer/*`, ...) — are appended as one JSON object per line, so runs on a
machine without network access keep their curves and `adana_b200.analysis` can work from files.  W&B, when
enabled, receives the identical dictionary.
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Dict, Iterable, List, Optional


def _plain(v):
    if hasattr(v, "item"):
        try:
            v = v.item()
        except Exception:
            return None
    if isinstance(v, bool):
        return v
    if isinstance(v, (int, str)):
        return v
    if isinstance(v, float):
        return v if math.isfinite(v) else None
    return None          # images, tables, histograms go to W&B only


class MetricsSink:
    def __init__(self, exp_dir, wandb_module=None, enabled: bool = True):
        self.path = Path(exp_dir) / "metrics.jsonl"
        self.wandb = wandb_module
        self.enabled = enabled
        if enabled:
            self.path.parent.mkdir(parents=True, exist_ok=True)

    def log(self, record: Dict, step: Optional[int] = None):
        if not self.enabled:
            return
        row = {k: _plain(v) for k, v in record.items()}
        row = {k: v for k, v in row.items() if v is not None}
        if step is not None:
            row.setdefault("iter", step)
        with open(self.path, "a") as f:
            f.write(json.dumps(row) + "\n")
        if self.wandb is not None:
            self.wandb.log(record, step=step)


def read_metrics(exp_dir_or_file) -> List[Dict]:
    p = Path(exp_dir_or_file)
    if p.is_dir():
        p = p / "metrics.jsonl"
    rows = []
    with open(p) as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append(json.loads(line))
    return rows


def series(rows: Iterable[Dict], key: str, x: str = "iter"):
    """-> (xs, ys) of every record that carries `key`."""
    xs, ys = [], []
    for r in rows:
        if key in r and x in r:
            xs.append(r[x])
            ys.append(r[key])
    return xs, ys
