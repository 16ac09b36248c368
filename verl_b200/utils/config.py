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
        v = yaml.safe_load(s)
    except yaml.YAMLError:
        return s
    if isinstance(v, str):
        # YAML 1.1 does not read "1e-6" as a number (it wants "1.0e-6"); launch scripts write it that way
        try:
            return float(v) if any(c in v for c in "eE.") and v.lower() not in ("nan", "inf", "-inf", ".", "e") else v
        except ValueError:
            return v
    return v


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


_CHOICE_RE = None


def _split_group_overrides(overrides: Sequence[str], config_dir: str) -> tuple[dict, list]:
    """Command-line items that choose a config GROUP member rather than set a value: ``model_engine=megatron`` or
    ``actor@actor_rollout_ref.actor=megatron_actor``. An item counts as a group choice when ``<config_dir>/<group>/`` exists
    and the key has no dot outside an ``@target``. Returns ({group or group@target: name}, remaining value overrides)."""
    choices, rest = {}, []
    for ov in overrides or []:
        if "=" in ov and not ov.startswith(("+", "~")):
            key, val = ov.split("=", 1)
            group = key.split("@", 1)[0]
            if "." not in group and os.path.isdir(os.path.join(config_dir, group)):
                choices[key] = val
                continue
        rest.append(ov)
    return choices, rest


def _load_yaml_with_defaults(path: str, choices: Optional[dict] = None, root_dir: Optional[str] = None, selected: Optional[dict] = None) -> dict:
    """Compose one yaml file with its ``defaults`` list (the subset of Hydra's semantics the config tree uses):

    * ``- name``                      merge ``<dir>/name.yaml`` at this file's root;
    * ``- group: name``               merge ``<dir>/group/name.yaml`` under key ``group`` and remember the choice, so that later
                                      entries (and files) may say ``${group}`` in a member name;
    * ``- group@a.b: name``           merge it under ``a.b`` instead;
    * ``- ../group@a: name``          group directory relative to this file's directory (used inside group files);
    * ``- _self_``                    where this file's own keys go (default: last);
    * ``choices`` (from the command line) replace the member name of a ``group`` / ``group@target`` entry.
    """
    choices = choices or {}
    selected = selected if selected is not None else {}
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    defaults = data.pop("defaults", None)
    if not defaults:
        return data
    root: dict = {}
    base_dir = os.path.dirname(path)
    root_dir = root_dir or base_dir
    merged_self = False

    def member(name) -> str:
        name = str(name)
        for g, v in selected.items():
            name = name.replace("${" + g + "}", str(v))
        return name

    for entry in defaults:
        if entry == "_self_":
            _merge(root, data)
            merged_self = True
            continue
        if isinstance(entry, str):
            _merge(root, _load_yaml_with_defaults(os.path.join(base_dir, f"{member(entry)}.yaml"), choices, root_dir, selected))
            continue
        (k, name), = entry.items()
        group, _, target = k.partition("@")
        name = choices.get(k, choices.get(os.path.basename(group), name))      # `group@target=x` or plain `group=x`
        if name is None or name == "null":
            continue
        name = member(name)
        gdir = os.path.normpath(os.path.join(base_dir, group))
        gname = os.path.basename(gdir)
        if not target:
            selected[gname] = name
        sub = _load_yaml_with_defaults(os.path.join(gdir, f"{name}.yaml"), choices, root_dir, selected)
        node = root
        if target:
            for p in target.split("."):
                node = node.setdefault(p, {})
            _merge(node, sub)
        elif isinstance(sub, dict) and set(sub.keys()) == {gname} and not isinstance(sub[gname], dict):
            root[gname] = sub[gname]          # a pure selector file such as ``model_engine: dp``
        else:
            _merge(root.setdefault(gname, {}), sub)
    if not merged_self:
        _merge(root, data)
    return root


_MISSING = "???"


def resolve_interpolations(root: dict) -> dict:
    """Replace ``${a.b.c}`` (absolute), ``${.sibling}`` / ``${..uncle}`` (relative to the node holding the value) and
    ``${oc.select:a.b,default}`` (value or default when the path is absent or null) references, after overrides were applied."""
    import re

    pat = re.compile(r"\$\{((?:[^${}]|\$\{[^${}]*\})+)\}")

    def walk_to(path_parts):
        cur: Any = root
        for part in path_parts:
            cur = cur[part]
        return cur

    def lookup(expr: str, here: tuple, depth: int):
        if depth > 20:
            raise ValueError("interpolation cycle in config")
        expr = expr.strip()
        if expr.startswith("oc.select:"):
            body = expr[len("oc.select:"):]
            path, _, default = body.partition(",")
            try:
                v = lookup(path.strip(), here, depth + 1)
            except (KeyError, TypeError, IndexError):
                v = None
            if v is None or v == _MISSING:
                d = default.strip()
                if not _:
                    return None
                return resolve(_parse_value(d) if not d.startswith("${") else d, here, depth + 1)
            return v
        if expr.startswith("."):
            up = len(expr) - len(expr.lstrip("."))
            base = here[:len(here) - (up - 1)] if up - 1 <= len(here) else ()
            parts = tuple(base) + tuple(x for x in expr.lstrip(".").split(".") if x)
        else:
            parts = tuple(expr.split("."))
        return resolve(walk_to(parts), parts[:-1], depth + 1)

    def resolve(v, here: tuple, depth=0):
        if isinstance(v, str) and "${" in v:
            m = pat.fullmatch(v.strip())
            if m:
                return lookup(m.group(1), here, depth)
            return pat.sub(lambda mm: str(lookup(mm.group(1), here, depth)), v)
        return v

    def walk(node, here: tuple):
        if isinstance(node, dict):
            for k in list(node.keys()):
                node[k] = walk(node[k], here + (k,)) if isinstance(node[k], (dict, list)) else resolve(node[k], here)
            return node
        if isinstance(node, list):
            return [walk(x, here) if isinstance(x, (dict, list)) else resolve(x, here[:-1] if False else here) for x in node]
        return resolve(node, here)

    return walk(root, ())


# spellings of the reference's tree that differ from this one's, rewritten on the command line
_OVERRIDE_ALIASES = (("critic.fsdp.", "critic.fsdp_config."), ("distillation.", "actor_rollout_ref.distillation."),
                     ("reward.reward_manager.name=", "reward.reward_manager="))


def _alias_override(ov: str) -> str:
    lead = ov[:len(ov) - len(ov.lstrip("+~"))]
    body = ov[len(lead):]
    for old, new in _OVERRIDE_ALIASES:
        if body.startswith(old):
            return lead + new + body[len(old):]
    return ov


def load_config(path_or_name: str = "ppo_trainer", overrides: Optional[Sequence[str]] = None, config_dir: Optional[str] = None) -> Config:
    if not os.path.exists(path_or_name):
        config_dir = config_dir or os.path.join(os.path.dirname(os.path.dirname(__file__)), "trainer", "config")
        path_or_name = os.path.join(config_dir, f"{path_or_name}.yaml")
    config_dir = config_dir or os.path.dirname(os.path.abspath(path_or_name))
    choices, values = _split_group_overrides([_alias_override(o) for o in (overrides or [])], config_dir)
    data = _load_yaml_with_defaults(path_or_name, choices)
    apply_overrides(data, values)
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
