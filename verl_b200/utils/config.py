"""Configuration tree: yaml files composed with a ``defaults`` list and dotted command-line overrides, exposed as
a dict with attribute access, plus conversion to typed dataclasses and cross-field validation.

Stands in for Hydra + OmegaConf of the reference (``verl/trainer/main_ppo.py:166-171``, ``verl/utils/config.py:23-250``)
which are not available offline; the key schema of ``ppo_trainer.yaml`` is kept so reference launch scripts'
``a.b.c=value`` overrides work unchanged.
"""

from __future__ import annotations

import copy
import dataclasses
import importlib
import os
from typing import Any, Optional, Sequence

import yaml

__all__ = ["Config", "load_config", "apply_overrides", "omega_conf_to_dataclass", "validate_config", "to_container", "resolve_interpolations"]


class Config(dict):
    """dict with attribute access; nested dicts are wrapped on the fly."""

    def __init__(self, data: Optional[dict] = None):
        super().__init__()
        for k, v in (data or {}).items():
            self[k] = v

    @staticmethod
    def _wrap(v):
        if isinstance(v, dict) and not isinstance(v, Config):
            return Config(v)
        if isinstance(v, list):
            return [Config._wrap(x) for x in v]
        return v

    def __setitem__(self, k, v):
        super().__setitem__(k, self._wrap(v))

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = v

    def __deepcopy__(self, memo):
        return Config(copy.deepcopy(dict(self), memo))

    def get(self, k, default=None):
        v = super().get(k, default)
        return default if v is None and default is not None else v

    def select(self, dotted: str, default=None):
        cur: Any = self
        for part in dotted.split("."):
            if not isinstance(cur, dict) or part not in cur:
                return default
            cur = cur[part]
        return cur


def to_container(cfg) -> Any:
    if isinstance(cfg, dict):
        return {k: to_container(v) for k, v in cfg.items()}
    if isinstance(cfg, (list, tuple)):
        return [to_container(v) for v in cfg]
    if dataclasses.is_dataclass(cfg) and not isinstance(cfg, type):
        return {f.name: to_container(getattr(cfg, f.name)) for f in dataclasses.fields(cfg)}
    return cfg


def _parse_value(s: str):
    try:
        return yaml.safe_load(s)
    except yaml.YAMLError:
        return s


def _merge(base: dict, extra: dict) -> dict:
    for k, v in extra.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            _merge(base[k], v)
        else:
            base[k] = copy.deepcopy(v)
    return base


def _set_path(root: dict, dotted: str, value, create: bool):
    parts = dotted.split(".")
    cur = root
    for p in parts[:-1]:
        if p not in cur or not isinstance(cur[p], dict):
            if not create and p not in cur:
                raise KeyError(f"override '{dotted}': key '{p}' does not exist (prefix with '+' to add it)")
            cur[p] = {} if not isinstance(cur.get(p), dict) else cur[p]
        cur = cur[p]
    if not create and parts[-1] not in cur:
        raise KeyError(f"override '{dotted}': key '{parts[-1]}' does not exist (prefix with '+' to add it)")
    cur[parts[-1]] = value


def apply_overrides(cfg: dict, overrides: Sequence[str]) -> dict:
    """``a.b=1`` sets an existing key, ``+a.b=1`` adds, ``++a.b=1`` sets-or-adds, ``~a.b`` deletes."""
    for ov in overrides or []:
        if ov.startswith("~"):
            parts = ov[1:].split("=")[0].split(".")
            cur = cfg
            for p in parts[:-1]:
                cur = cur[p]
            cur.pop(parts[-1], None)
            continue
        create = False
        while ov.startswith("+"):
            create = True
            ov = ov[1:]
        if "=" not in ov:
            raise ValueError(f"malformed override '{ov}'")
        key, val = ov.split("=", 1)
        _set_path(cfg, key, _parse_value(val), create)
    return cfg


def _load_yaml_with_defaults(path: str, seen=None) -> dict:
    """``defaults:`` entries ``group@target.path: name`` load ``<dir>/<group>/<name>.yaml`` under ``target.path``;
    ``_self_`` marks where this file's own keys are merged."""
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    defaults = data.pop("defaults", None)
    if not defaults:
        return data
    root: dict = {}
    base_dir = os.path.dirname(path)
    merged_self = False
    for entry in defaults:
        if entry == "_self_":
            _merge(root, data)
            merged_self = True
            continue
        if isinstance(entry, dict):
            (k, name), = entry.items()
            group, _, target = k.partition("@")
            sub = _load_yaml_with_defaults(os.path.join(base_dir, group, f"{name}.yaml"))
            node = root
            if target:
                for p in target.split("."):
                    node = node.setdefault(p, {})
            else:
                node = root.setdefault(group, {})
            _merge(node, sub)
    if not merged_self:
        _merge(root, data)
    return root


def resolve_interpolations(root: dict) -> dict:
    """Replace ``${a.b.c}`` references (OmegaConf style) by the value they point at, after overrides were applied."""
    import re

    pat = re.compile(r"\$\{([^}]+)\}")

    def lookup(path: str, depth=0):
        cur: Any = root
        for part in path.split("."):
            cur = cur[part]
        return resolve(cur, depth + 1)

    def resolve(v, depth=0):
        if depth > 20:
            raise ValueError("interpolation cycle in config")
        if isinstance(v, str):
            m = pat.fullmatch(v.strip())
            if m:
                return lookup(m.group(1), depth)
            return pat.sub(lambda mm: str(lookup(mm.group(1), depth)), v)
        return v

    def walk(node):
        if isinstance(node, dict):
            for k in list(node.keys()):
                node[k] = walk(node[k])
            return node
        if isinstance(node, list):
            return [walk(x) for x in node]
        return resolve(node)

    return walk(root)


def load_config(path_or_name: str = "ppo_trainer", overrides: Optional[Sequence[str]] = None, config_dir: Optional[str] = None) -> Config:
    if not os.path.exists(path_or_name):
        config_dir = config_dir or os.path.join(os.path.dirname(os.path.dirname(__file__)), "trainer", "config")
        path_or_name = os.path.join(config_dir, f"{path_or_name}.yaml")
    data = _load_yaml_with_defaults(path_or_name)
    apply_overrides(data, overrides or [])
    resolve_interpolations(data)
    return Config(data)


def omega_conf_to_dataclass(config, dataclass_type=None):
    """Instantiate the dataclass named by ``_target_`` (or ``dataclass_type``) from a config node, recursively."""
    if config is None:
        return None
    if dataclasses.is_dataclass(config) and not isinstance(config, type):
        return config
    if not isinstance(config, dict):
        return config
    if dataclass_type is None:
        target = config.get("_target_")
        if not target:
            return config
        mod, _, name = target.rpartition(".")
        mod = mod.replace("verl.", "verl_b200.", 1) if mod.startswith("verl.") else mod
        dataclass_type = getattr(importlib.import_module(mod), name)
    names = {f.name: f for f in dataclasses.fields(dataclass_type)}
    kwargs = {}
    for k, v in config.items():
        if k == "_target_" or k not in names:
            continue
        if isinstance(v, dict) and v.get("_target_"):
            v = omega_conf_to_dataclass(v)
        kwargs[k] = v
    return dataclass_type(**kwargs)


def validate_config(config: Config, use_reference_policy: bool = False, use_critic: bool = False) -> None:
    """Cross-field checks the reference performs before training (``verl/utils/config.py:120-250``)."""
    n_gpus = config.trainer.n_gpus_per_node * config.trainer.nnodes
    ar = config.actor_rollout_ref
    actor, rollout = ar.actor, ar.rollout
    real_bsz = config.data.train_batch_size * rollout.n
    if actor.strategy in ("fsdp", "fsdp2"):
        sp = actor.get("fsdp_config", {}).get("ulysses_sequence_parallel_size", 1) or 1
        dp = n_gpus // sp
        assert n_gpus % sp == 0, f"n_gpus ({n_gpus}) must be divisible by ulysses_sequence_parallel_size ({sp})"
        assert real_bsz % dp == 0, f"train_batch_size*n ({real_bsz}) must be divisible by the data-parallel size ({dp})"
        if sp > 1:
            assert ar.model.get("use_remove_padding", True), "Ulysses sequence parallelism requires use_remove_padding"
    elif actor.strategy == "megatron":
        m = actor.megatron
        mp = m.tensor_model_parallel_size * m.pipeline_model_parallel_size * m.get("context_parallel_size", 1)
        assert n_gpus % mp == 0, f"n_gpus ({n_gpus}) must be divisible by tp*pp*cp ({mp})"
        assert real_bsz % (n_gpus // mp) == 0, "train_batch_size*n must be divisible by the data-parallel size"

    def check_mutually_exclusive(mbs, mbs_per_gpu, name):
        if mbs is None and mbs_per_gpu is None:
            raise ValueError(f"[{name}] set either '{name}.micro_batch_size' or '{name}.micro_batch_size_per_gpu'")
        if mbs is not None and mbs_per_gpu is not None:
            raise ValueError(f"[{name}] 'micro_batch_size' and 'micro_batch_size_per_gpu' are mutually exclusive; "
                             "the former is deprecated")

    if not actor.get("use_dynamic_bsz", False):
        check_mutually_exclusive(actor.get("ppo_micro_batch_size"), actor.get("ppo_micro_batch_size_per_gpu"), "actor_rollout_ref.actor")
        assert config.data.train_batch_size >= actor.ppo_mini_batch_size, "train_batch_size must be >= ppo_mini_batch_size"
        if use_reference_policy and not ar.ref.get("log_prob_use_dynamic_bsz", False):
            check_mutually_exclusive(ar.ref.get("log_prob_micro_batch_size"), ar.ref.get("log_prob_micro_batch_size_per_gpu"), "actor_rollout_ref.ref")
    if actor.get("loss_agg_mode", "token-mean") not in ("token-mean", "token-sum", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"):
        raise ValueError(f"Invalid loss_agg_mode: {actor.loss_agg_mode}")
    if config.algorithm.get("use_kl_in_reward", False) and actor.get("use_kl_loss", False):
        print("NOTICE: both in-reward KL and KL loss are enabled.")
    if use_critic and not config.critic.get("use_dynamic_bsz", False):
        check_mutually_exclusive(config.critic.get("ppo_micro_batch_size"), config.critic.get("ppo_micro_batch_size_per_gpu"), "critic")
    if config.data.get("val_batch_size") is not None:
        print("WARNING: val_batch_size is deprecated; validation data is sent to the rollout engine in one batch.")
    if rollout.get("val_kwargs", {}).get("do_sample", False):
        assert rollout.temperature > 0, "validation sampling requires temperature > 0"
    lora_rank = ar.model.get("lora_rank", 0) or 0
    if lora_rank > 0 and actor.strategy not in ("fsdp", "fsdp2", "megatron"):
        raise ValueError("LoRA requires the fsdp or megatron strategy")
    print("[validate_config] All configuration checks passed successfully!")
