"""Experiment tracking fan-out.

Parity target: ``verl/utils/tracking.py`` (``Tracking`` :37-220 with its back-end list, ``ValidationGenerationsLogger``
:548).  Back-ends whose client library is not installed raise at construction, like the reference.
"""

from __future__ import annotations

import dataclasses
import json
import os
from enum import Enum
from pathlib import Path
from typing import Any, Optional

__all__ = ["Tracking", "ValidationGenerationsLogger", "compute_data_metrics_flat"]


def _flatten(d, prefix: str = "", sep: str = "/") -> dict:
    out = {}
    for k, v in (d.items() if hasattr(d, "items") else []):
        key = f"{prefix}{sep}{k}" if prefix else str(k)
        if hasattr(v, "items"):
            out.update(_flatten(v, key, sep))
        else:
            out[key] = v
    return out


def _plain(obj):
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: _plain(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
    if hasattr(obj, "items"):
        return {str(k): _plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_plain(v) for v in obj]
    if isinstance(obj, Enum):
        return f"{obj.__class__.__name__}.{obj.name}"
    if isinstance(obj, Path):
        return str(obj)
    if isinstance(obj, (int, float, str, bool)) or obj is None:
        return obj
    return str(obj)


compute_data_metrics_flat = _flatten


class _Console:
    def __init__(self, print_to_console: bool = True):
        self.on = print_to_console

    def log(self, data: dict, step: int) -> None:
        if self.on:
            body = " - ".join(f"{k}:{v:.4g}" if isinstance(v, float) else f"{k}:{v}" for k, v in sorted(data.items()))
            print(f"step:{step} - {body}", flush=True)

    def finish(self):
        pass


class _FileLogger:
    def __init__(self, project_name: str, experiment_name: str):
        root = os.environ.get("VERL_FILE_LOGGER_ROOT", os.path.expanduser("~/verl_logs"))
        path = os.environ.get("VERL_FILE_LOGGER_PATH") or os.path.join(root, project_name, f"{experiment_name}.jsonl")
        os.makedirs(os.path.dirname(path), exist_ok=True)
        self.path = path
        self.fp = open(path, "a")

    def log(self, data: dict, step: int) -> None:
        self.fp.write(json.dumps({"step": step, "data": _plain(data)}) + "\n")
        self.fp.flush()

    def finish(self):
        self.fp.close()


class _TensorBoard:
    def __init__(self, project_name: str, experiment_name: str):
        from torch.utils.tensorboard import SummaryWriter

        d = os.environ.get("TENSORBOARD_DIR", f"tensorboard_log/{project_name}/{experiment_name}")
        os.makedirs(d, exist_ok=True)
        self.w = SummaryWriter(d)

    def log(self, data: dict, step: int) -> None:
        for k, v in data.items():
            if isinstance(v, (int, float)):
                self.w.add_scalar(k, v, step)

    def finish(self):
        self.w.close()


class _ModuleBackend:
    """wandb-compatible clients (wandb, swanlab, trackio): ``init`` then ``log(data, step=)``."""

    def __init__(self, module_name: str, project_name: str, experiment_name: str, config):
        import importlib

        self.m = importlib.import_module(module_name)
        kw = dict(project=project_name, name=experiment_name, config=_plain(config) if config is not None else None)
        if module_name == "wandb" and os.environ.get("WANDB_MODE") is None and not os.environ.get("WANDB_API_KEY"):
            kw["mode"] = "offline"
        self.run = self.m.init(**kw)

    def log(self, data: dict, step: int) -> None:
        self.m.log(data, step=step)

    def finish(self):
        try:
            self.m.finish()
        except Exception:
            pass


class _MLflow:
    def __init__(self, project_name: str, experiment_name: str, config):
        import mlflow

        self.mlflow = mlflow
        uri = os.environ.get("MLFLOW_TRACKING_URI", "sqlite:////tmp/mlruns.db")
        mlflow.set_tracking_uri(uri)
        mlflow.set_experiment(project_name)
        mlflow.start_run(run_name=experiment_name)
        if config is not None:
            mlflow.log_params({k: str(v)[:250] for k, v in _flatten(_plain(config)).items()})

    def log(self, data: dict, step: int) -> None:
        self.mlflow.log_metrics({k.replace("@", "_at_"): float(v) for k, v in data.items() if isinstance(v, (int, float))}, step=step)

    def finish(self):
        self.mlflow.end_run()


class _ClearML:
    def __init__(self, project_name: str, experiment_name: str, config):
        import clearml

        self.task = clearml.Task.init(task_name=experiment_name, project_name=project_name, continue_last_task=True,
                                      output_uri=False)
        if config is not None:
            self.task.connect_configuration(_plain(config), name="Hyperparameters")

    def log(self, data: dict, step: int) -> None:
        lg = self.task.get_logger()
        for k, v in data.items():
            title, _, series = k.partition("/")
            if isinstance(v, (int, float)):
                lg.report_scalar(title=title, series=series or title, value=v, iteration=step)

    def finish(self):
        self.task.close()


class Tracking:
    supported_backend = ["wandb", "mlflow", "swanlab", "vemlp_wandb", "tensorboard", "console", "clearml", "trackio",
                         "file", "rl_insight"]

    def __init__(self, project_name: str, experiment_name: str, default_backend="console", config=None):
        if isinstance(default_backend, str):
            default_backend = [default_backend]
        for b in default_backend:
            assert b in self.supported_backend, f"{b} is not supported"
        self.logger: dict[str, Any] = {}
        for b in default_backend:
            if b == "console":
                self.logger[b] = _Console()
            elif b == "file":
                self.logger[b] = _FileLogger(project_name, experiment_name)
            elif b == "tensorboard":
                self.logger[b] = _TensorBoard(project_name, experiment_name)
            elif b in ("wandb", "swanlab", "trackio"):
                self.logger[b] = _ModuleBackend(b, project_name, experiment_name, config)
            elif b == "vemlp_wandb":
                self.logger[b] = _ModuleBackend("volcengine_ml_platform.wandb", project_name, experiment_name, config)
            elif b == "mlflow":
                self.logger[b] = _MLflow(project_name, experiment_name, config)
            elif b == "clearml":
                self.logger[b] = _ClearML(project_name, experiment_name, config)
            elif b == "rl_insight":
                self.logger[b] = _FileLogger(project_name, experiment_name + ".rl_insight")

    def log(self, data: dict, step: int, backend=None) -> None:
        for name, lg in self.logger.items():
            if backend is None or name in backend:
                lg.log(data=data, step=step)

    def __del__(self):
        for lg in getattr(self, "logger", {}).values():
            try:
                lg.finish()
            except Exception:
                pass


class ValidationGenerationsLogger:
    """Logs (input, output, score) triples of validation samples to the configured back-ends or a JSONL file."""

    def __init__(self, project_name: Optional[str] = None, experiment_name: Optional[str] = None):
        self.project_name, self.experiment_name = project_name, experiment_name

    def log(self, loggers, samples: list, step: int) -> None:
        loggers = [loggers] if isinstance(loggers, str) else list(loggers or [])
        if "wandb" in loggers:
            import wandb

            cols = ["step"] + sum([[f"input_{i+1}", f"output_{i+1}", f"score_{i+1}"] for i in range(len(samples))], [])
            table = wandb.Table(columns=cols)
            table.add_data(step, *[x for s in samples for x in s])
            wandb.log({"val/generations": table}, step=step)
        if "file" in loggers or "console" in loggers:
            root = os.environ.get("VERL_FILE_LOGGER_ROOT", os.path.expanduser("~/verl_logs"))
            path = os.path.join(root, self.project_name or "verl_b200", f"{self.experiment_name or 'run'}.val_generations.jsonl")
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "a") as f:
                for s in samples:
                    f.write(json.dumps({"step": step, "input": s[0], "output": s[1], "score": s[2]}) + "\n")
