"""Experiment tracking fan-out: console, jsonl file, tensorboard, wandb, mlflow (each optional).

Parity target: ``verl/utils/tracking.py`` (Tracking :38, FileLogger :529, ValidationGenerationsLogger :664) and
``verl/utils/logger/aggregate_logger.py`` (LocalLogger).
"""

from __future__ import annotations

import json
import numbers
import os
import time
from typing import Any, Optional

__all__ = ["Tracking", "LocalLogger", "FileLogger", "ValidationGenerationsLogger", "concat_dict_to_str"]


def concat_dict_to_str(d: dict, step: int) -> str:
    parts = [f"step:{step}"]
    for k, v in d.items():
        if isinstance(v, numbers.Number):
            parts.append(f"{k}:{v:.6g}")
    return " - ".join(parts)


class LocalLogger:
    def __init__(self, print_to_console: bool = True):
        self.print_to_console = print_to_console

    def log(self, data, step):
        if self.print_to_console:
            print(concat_dict_to_str(data, step), flush=True)

    def finish(self):
        pass


class FileLogger:
    """One json object per step under ``$VERL_FILE_LOGGER_PATH`` or ``$VERL_FILE_LOGGER_ROOT/<project>/<experiment>.jsonl``."""

    def __init__(self, project_name: str, experiment_name: str):
        path = os.getenv("VERL_FILE_LOGGER_PATH")
        if path is None:
            root = os.path.expanduser(os.getenv("VERL_FILE_LOGGER_ROOT", "."))
            d = os.path.join(root, project_name)
            os.makedirs(d, exist_ok=True)
            path = os.path.join(d, f"{experiment_name}.jsonl")
        else:
            os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
        self.filepath = path
        self.fp = open(path, "w")

    def log(self, data, step):
        self.fp.write(json.dumps({"step": step, "data": {k: v for k, v in data.items() if isinstance(v, (numbers.Number, str))}}) + "\n")
        self.fp.flush()

    def finish(self):
        self.fp.close()


class _TensorboardAdapter:
    def __init__(self, project_name, experiment_name):
        from torch.utils.tensorboard import SummaryWriter

        d = os.environ.get("TENSORBOARD_DIR", f"tensorboard_log/{project_name}/{experiment_name}")
        os.makedirs(d, exist_ok=True)
        self.writer = SummaryWriter(d)

    def log(self, data, step):
        for k, v in data.items():
            if isinstance(v, numbers.Number):
                self.writer.add_scalar(k, v, step)

    def finish(self):
        self.writer.close()


class Tracking:
    supported_backend = ["wandb", "mlflow", "swanlab", "vemlp_wandb", "tensorboard", "console", "clearml", "trackio", "file", "rl_insight"]

    def __init__(self, project_name: str, experiment_name: str, default_backend="console", config: Optional[dict] = None):
        if isinstance(default_backend, str):
            default_backend = [default_backend]
        for b in default_backend:
            assert b in self.supported_backend, f"{b} is not supported"
        self.logger: dict[str, Any] = {}
        if "console" in default_backend:
            self.logger["console"] = LocalLogger(True)
        if "file" in default_backend:
            self.logger["file"] = FileLogger(project_name, experiment_name)
        if "tensorboard" in default_backend:
            self.logger["tensorboard"] = _TensorboardAdapter(project_name, experiment_name)
        if "wandb" in default_backend:
            import wandb

            wandb.init(project=project_name, name=experiment_name, config=config, mode=os.environ.get("WANDB_MODE", "offline"))
            self.logger["wandb"] = wandb
        if "mlflow" in default_backend:
            import mlflow

            mlflow.start_run(run_name=experiment_name)
            self.logger["mlflow"] = _MlflowAdapter(mlflow)
        for b in default_backend:
            if b not in self.logger:
                raise ImportError(f"tracking backend '{b}' needs an SDK that is not installed in this environment")

    def log(self, data: dict, step: int, backend=None):
        for name, inst in self.logger.items():
            if backend is None or name in backend:
                inst.log(data=data, step=step)

    def __del__(self):
        for name, inst in getattr(self, "logger", {}).items():
            try:
                inst.finish()
            except Exception:
                pass


class _MlflowAdapter:
    def __init__(self, mlflow):
        self.mlflow = mlflow

    def log(self, data, step):
        self.mlflow.log_metrics({k.replace("@", "_at_"): v for k, v in data.items() if isinstance(v, numbers.Number)}, step=step)

    def finish(self):
        self.mlflow.end_run()


class ValidationGenerationsLogger:
    """Dump (input, output, score) triples of validation samples to jsonl (console/file backends) or a wandb table."""

    def __init__(self, project_name: str = None, experiment_name: str = None):
        self.project_name, self.experiment_name = project_name, experiment_name

    def log(self, loggers, samples, step):
        path = os.path.join(os.getenv("VERL_FILE_LOGGER_ROOT", "."), f"val_generations_{self.experiment_name or 'run'}.jsonl")
        with open(path, "a") as f:
            for inp, out, score in samples:
                f.write(json.dumps({"step": step, "input": inp, "output": out, "score": score}) + "\n")
