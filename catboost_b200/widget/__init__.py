"""Training-curve viewers (the ``catboost.widget`` names: ``MetricVisualizer``, ``MetricsPlotter``).

The reference draws live curves with an ipywidgets front end and plotly
(catboost/python-package/catboost/widget/ipythonwidget.py, metrics_plotter.py).  Here the data side is complete and
headless: ``MetricVisualizer`` reads the ``catboost_training.json`` / ``*_error.tsv`` logs that ``fit`` writes into its
train directories and hands back the curves (``curves()``), renders them as text (``to_text()``), or, when plotly is
importable, as one figure per metric (``figures()``); ``start()`` shows the figures in a notebook and falls back to the
text rendering elsewhere.  ``MetricsPlotter`` collects values pushed iteration by iteration (the callback interface of
the reference's plotter) and renders the same way.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

from ..data.pool import CatBoostError

__all__ = ["MetricVisualizer", "MetricsPlotter"]


def _read_train_dir(path: str) -> Dict[str, Dict[str, List[float]]]:
    """{'learn' | 'test' | ...: {metric: values}} from a train directory's json log (tsv logs as a fallback)."""
    out: Dict[str, Dict[str, List[float]]] = {}
    js = os.path.join(path, "catboost_training.json")
    if os.path.exists(js):
        with open(js) as fh:
            doc = json.load(fh)
        meta = doc.get("meta", {})
        for part, key in (("learn", "learn_metrics"), ("test", "test_metrics")):
            names = [m["name"] if isinstance(m, dict) else str(m) for m in meta.get(key, [])]
            for it in doc.get("iterations", []):
                vals = it.get(part)
                if vals is None:
                    continue
                for nm, v in zip(names, vals):
                    out.setdefault(part, {}).setdefault(nm, []).append(float(v))
        if out:
            return out
    for part in ("learn", "test"):
        tsv = os.path.join(path, f"{part}_error.tsv")
        if not os.path.exists(tsv):
            continue
        with open(tsv) as fh:
            head = fh.readline().rstrip("\n").split("\t")[1:]
            for line in fh:
                cells = line.rstrip("\n").split("\t")[1:]
                for nm, v in zip(head, cells):
                    out.setdefault(part, {}).setdefault(nm, []).append(float(v))
    return out


def _render_text(curves: Dict[str, Dict[str, Dict[str, List[float]]]], width: int = 60) -> str:
    """One line per (run, part, metric): first / best / last value and a coarse sparkline."""
    marks = " .:-=+*#%@"
    lines = []
    for run, parts in curves.items():
        for part, metrics in parts.items():
            for nm, vals in metrics.items():
                if not vals:
                    continue
                lo, hi = min(vals), max(vals)
                step = max(1, len(vals) // width)
                pts = vals[::step][:width]
                spark = "".join(marks[int((v - lo) / (hi - lo) * (len(marks) - 1))] if hi > lo else marks[0] for v in pts)
                lines.append(f"{run} {part} {nm}: first {vals[0]:.6g} min {lo:.6g} max {hi:.6g} last {vals[-1]:.6g} |{spark}|")
    return "\n".join(lines)


class MetricVisualizer:
    def __init__(self, train_dirs, subdirs: bool = False):
        if isinstance(train_dirs, (str, os.PathLike)):
            train_dirs = [train_dirs]
        dirs = [os.fspath(d) for d in train_dirs]
        if subdirs:
            dirs = [os.path.join(d, s) for d in dirs for s in sorted(os.listdir(d)) if os.path.isdir(os.path.join(d, s))]
        if not dirs:
            raise CatBoostError("no train directories given")
        self.train_dirs = dirs

    def curves(self) -> Dict[str, Dict[str, Dict[str, List[float]]]]:
        """{train dir: {'learn' | 'test': {metric: values per logged iteration}}}."""
        return {d: _read_train_dir(d) for d in self.train_dirs}

    def to_text(self) -> str:
        return _render_text(self.curves())

    def figures(self):
        """One plotly figure per metric with a trace per (train dir, learn / test)."""
        try:
            import plotly.graph_objects as go
        except ImportError as e:
            raise CatBoostError("figures() needs the plotly package") from e
        by_metric: Dict[str, list] = {}
        for d, parts in self.curves().items():
            for part, metrics in parts.items():
                for nm, vals in metrics.items():
                    by_metric.setdefault(nm, []).append((f"{os.path.basename(d) or d} {part}", vals))
        figs = {}
        for nm, traces in by_metric.items():
            fig = go.Figure()
            for label, vals in traces:
                fig.add_trace(go.Scatter(y=vals, mode="lines", name=label))
            fig.update_layout(title=nm, xaxis_title="iteration")
            figs[nm] = fig
        return figs

    def start(self):
        """Shows the curves: plotly figures inside a notebook, the text rendering on a terminal."""
        try:
            from IPython import get_ipython
            in_notebook = get_ipython() is not None and "IPKernelApp" in get_ipython().config
        except Exception:
            in_notebook = False
        if in_notebook:
            try:
                for fig in self.figures().values():
                    fig.show()
                return
            except CatBoostError:
                pass
        print(self.to_text())


class MetricsPlotter:
    """Collects metric values as they are produced: ``plotter.log(epoch, train, {"loss": v})`` per iteration, as the
    reference's plotter is driven by its callbacks; ``train`` picks the learn or the validation series."""

    def __init__(self, train_metrics: Sequence, test_metrics: Optional[Sequence] = None, total_iterations: Optional[int] = None):
        name = lambda m: m["name"] if isinstance(m, dict) else str(m)
        self.train_metrics = [name(m) for m in train_metrics]
        self.test_metrics = [name(m) for m in (test_metrics if test_metrics is not None else train_metrics)]
        self.total_iterations = total_iterations
        self._data: Dict[str, Dict[str, List[float]]] = {"learn": {m: [] for m in self.train_metrics},
                                                          "test": {m: [] for m in self.test_metrics}}

    def log(self, epoch: int, train: bool, metrics: Dict[str, float]):
        part = self._data["learn" if train else "test"]
        for nm, v in metrics.items():
            if nm not in part:
                raise CatBoostError(f"metric {nm!r} was not declared")
            series = part[nm]
            if epoch < len(series):
                series[epoch] = float(v)
            else:
                series.extend([float("nan")] * (epoch - len(series)) + [float(v)])

    def curves(self):
        return {"run": self._data}

    def to_text(self) -> str:
        return _render_text(self.curves())
