"""Metric sinks (reference: src/zeroband/utils/metric_logger.py:6-49).

``DummyMetricLogger`` keeps a list of dicts and pickles it to the path named by ``project`` on
``finish()`` — tests read that file as their observation channel. ``WandbMetricLogger`` needs the
optional ``wandb`` package."""
from __future__ import annotations

import pickle
from typing import Any, Protocol


class MetricLogger(Protocol):
    def log(self, metrics: dict[str, Any]): ...
    def finish(self): ...


class WandbMetricLogger:
    def __init__(self, project, config, resume: bool):
        import wandb
        # the trainer passes {"config": <Config dump>, "world_info": ...}; the run name lives in the inner dict
        inner = config.get("config", config) if isinstance(config, dict) else {}
        run_name = inner.get("run_name") if isinstance(inner, dict) else None
        wandb.init(project=project, config=config, name=run_name, resume="auto" if resume else None)

    def log(self, metrics: dict[str, Any]):
        import wandb
        wandb.log(metrics)

    def finish(self):
        import wandb
        wandb.finish()


class DummyMetricLogger:
    def __init__(self, project, *args, **kwargs):
        self.project = project
        self.data: list[dict[str, Any]] = []

    def log(self, metrics: dict[str, Any]):
        self.data.append(dict(metrics))

    def finish(self):
        with open(self.project, "wb") as f:
            pickle.dump(self.data, f)
