"""Experiment tracking fan-out: console, jsonl file, tensorboard, wandb (+ the vemlp flavour), mlflow, swanlab, clearml,
trackio and rl_insight. Every SDK is imported only when its backend is selected.

Parity target: ``verl/utils/tracking.py`` (Tracking :38, FileLogger :529, ValidationGenerationsLogger :664) and
``verl/utils/logger/aggregate_logger.py`` (LocalLogger).
"""

from __future__ import annotations

import json
import numbers
import os
import time
from typing import Any, Optional

__all__ = ["Tracking", "LocalLogger", "FileLogger", "ClearMLLogger", "RLInsightLogger", "ValidationGenerationsLogger", "concat_dict_to_str"]


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
        if "vemlp_wandb" in default_backend:
            # volcengine ML platform: its wandb fork, credentials from the environment
            import volcengine_ml_platform
            from volcengine_ml_platform import wandb as vemlp_wandb

            volcengine_ml_platform.init(ak=os.environ["VOLC_ACCESS_KEY_ID"], sk=os.environ["VOLC_SECRET_ACCESS_KEY"], region=os.environ["MLP_TRACKING_REGION"])
            vemlp_wandb.init(project=project_name, name=experiment_name, config=config, sync_tensorboard=True)
            self.logger["vemlp_wandb"] = vemlp_wandb
        if "swanlab" in default_backend:
            import swanlab

            key = os.environ.get("SWANLAB_API_KEY")
            if key:
                swanlab.login(key)
            swanlab.init(project=project_name, experiment_name=experiment_name, config={"FRAMEWORK": "verl_b200", **(config or {})},
                         logdir=os.environ.get("SWANLAB_LOG_DIR", "swanlog"), mode=os.environ.get("SWANLAB_MODE", "cloud"))
            self.logger["swanlab"] = swanlab
        if "clearml" in default_backend:
            self.logger["clearml"] = ClearMLLogger(project_name, experiment_name, config)
        if "trackio" in default_backend:
            import trackio

            trackio.init(project=project_name, name=experiment_name, config=config)
            self.logger["trackio"] = _TrackioAdapter(trackio)
        if "rl_insight" in default_backend:
            self.logger["rl_insight"] = RLInsightLogger(project_name, experiment_name, config)
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


class _TrackioAdapter:
    def __init__(self, trackio):
        self.trackio = trackio

    def log(self, data, step):
        self.trackio.log(data, step=step)

    def finish(self):
        self.trackio.finish()


class ClearMLLogger:
    """One ClearML task per run; scalars are reported as (title, series) split at the first ``/`` of the metric name
    (reference: ``verl/utils/tracking.py:463-512``)."""

    def __init__(self, project_name: str, experiment_name: str, config=None):
        import clearml

        self._task = clearml.Task.init(task_name=experiment_name, project_name=project_name, continue_last_task=True, output_uri=False)
        if config is not None:
            self._task.connect_configuration(dict(config), name="Hyperparameters")

    def log(self, data, step):
        lg = self._task.get_logger()
        for k, v in data.items():
            if not isinstance(v, numbers.Number):
                continue
            title, _, series = k.partition("/")
            lg.report_scalar(title=title, series=series or title, value=float(v), iteration=step)

    def finish(self):
        self._task.close()


class RLInsightLogger:
    """Exports scalar metrics as gauges and runtime phases as traced states to ``rl_insight`` when the process opted in with
    ``VERL_RL_INSIGHT_ENABLE=1``; otherwise every call is a no-op, so call sites need no guard
    (reference: ``verl/utils/tracking.py:226-460``)."""

    ENABLE_ENV = "VERL_RL_INSIGHT_ENABLE"
    _module = None
    _started = False

    def __init__(self, project_name=None, experiment_name=None, config=None):
        self.init(project_name, experiment_name, config)

    @classmethod
    def enabled(cls) -> bool:
        return os.getenv(cls.ENABLE_ENV) == "1"

    @classmethod
    def _sdk(cls):
        if cls._module is None:
            import rl_insight

            cls._module = rl_insight
        return cls._module

    @classmethod
    def init(cls, project_name=None, experiment_name=None, config=None):
        if not cls.enabled() or cls._started:
            return
        sub = {}
        try:
            sub = (config or {}).get("trainer", {}).get("rl_insight", {}) or {}
        except (AttributeError, TypeError):
            pass
        cls._sdk().init(project=project_name, experiment_name=experiment_name, config=sub)
        cls._started = True

    @classmethod
    def log(cls, data, step):
        if not cls.enabled():
            return
        cls.init()
        gauge = cls._sdk().metric_gauge
        for k, v in data.items():
            try:
                gauge(str(k).replace("/", "_"), float(v))
            except (TypeError, ValueError):
                continue

    @classmethod
    def finish(cls):
        if cls._started:
            cls._sdk().finish()
            cls._started = False

    @classmethod
    def trace_state(cls, state_name: str, *, state_lane_id=None, **labels):
        """Context manager marking a runtime state (rollout, update, weight sync ...) on a lane of the timeline."""
        from contextlib import nullcontext

        if not cls.enabled():
            return nullcontext()
        cls.init()
        return cls._sdk().trace_state(state_name, state_lane_id=state_lane_id, **labels)


class ValidationGenerationsLogger:
    """Dump (input, output, score) triples of validation samples to jsonl (console/file backends) or a wandb table."""

    def __init__(self, project_name: str = None, experiment_name: str = None):
        self.project_name, self.experiment_name = project_name, experiment_name

    def log(self, loggers, samples, step):
        path = os.path.join(os.getenv("VERL_FILE_LOGGER_ROOT", "."), f"val_generations_{self.experiment_name or 'run'}.jsonl")
        with open(path, "a") as f:
            for inp, out, score in samples:
                f.write(json.dumps({"step": step, "input": inp, "output": out, "score": score}) + "\n")
        loggers = loggers or []
        text = "\n\n".join(f"input: {i}\n---\noutput: {o}\n---\nscore: {s}" for i, o, s in samples)
        if "swanlab" in loggers:
            import swanlab

            swanlab.log({"val/generations": [swanlab.Text(f"input: {i}\n---\noutput: {o}\n---\nscore: {s}", caption=f"sample {n + 1}")
                                             for n, (i, o, s) in enumerate(samples)]}, step=step)
        if "clearml" in loggers:
            import clearml

            task = clearml.Task.current_task()
            if task is not None:
                task.get_logger().report_text(text, print_console=False)
        if "trackio" in loggers:
            import trackio

            trackio.log({"val/generations": text}, step=step)
        if "tensorboard" in loggers and hasattr(self, "_tb_writer"):
            self._tb_writer.add_text("val/generations", text, step)
