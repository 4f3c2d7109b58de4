"""YAML configuration tree with Hydra-style composition, dotted overrides and interpolation.

Hydra/OmegaConf are not a dependency: this module implements the subset the trainer schema uses —
``defaults:`` lists (``group: option`` and ``group@target.path: option``), ``_self_`` ordering, dotted CLI
overrides (``a.b.c=value``, ``+a.b=value`` to add, ``~a.b`` to delete), ``${path.to.key}`` and
``${oc.select:key,default}`` interpolation, and ``_target_``-driven dataclass instantiation.

Parity target: ``verl/utils/config.py:23-202`` and the Hydra usage in ``verl/trainer/main_ppo.py:166``.
"""

from __future__ import annotations

import copy
import importlib
import os
import re
from dataclasses import fields, is_dataclass
from typing import Any, Iterable, Optional

import yaml

__all__ = ["DictConfig", "load_config", "apply_overrides", "omega_conf_to_dataclass", "update_dict_with_config",
           "validate_config", "to_container", "compose"]


class DictConfig(dict):
    """dict with attribute access and nested auto-wrapping."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        for k, v in dict(*args, **kwargs).items():
            self[k] = v

    @staticmethod
    def _wrap(v):
        if isinstance(v, dict) and not isinstance(v, DictConfig):
            return DictConfig(v)
        if isinstance(v, list):
            return [DictConfig._wrap(x) for x in v]
        return v

    def __setitem__(self, k, v):
        super().__setitem__(k, self._wrap(v))

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k) from None

    def __setattr__(self, k, v):
        self[k] = v

    def __delattr__(self, k):
        del self[k]

    def get(self, k, default=None):
        v = super().get(k, default)
        return default if v is None and default is not None else v

    def select(self, path: str, default=None):
        cur: Any = self
        for p in path.split("."):
            if isinstance(cur, dict) and p in cur:
                cur = cur[p]
            else:
                return default
        return cur

    def set_path(self, path: str, value) -> None:
        parts = path.split(".")
        cur = self
        for p in parts[:-1]:
            if p not in cur or not isinstance(cur[p], dict):
                cur[p] = DictConfig()
            cur = cur[p]
        cur[parts[-1]] = value

    def __deepcopy__(self, memo):
        return DictConfig({k: copy.deepcopy(v, memo) for k, v in self.items()})


def to_container(cfg) -> Any:
    if isinstance(cfg, dict):
        return {k: to_container(v) for k, v in cfg.items()}
    if isinstance(cfg, list):
        return [to_container(v) for v in cfg]
    return cfg


_NUM = re.compile(r"^[+-]?(\d+\.?\d*|\.\d+)([eE][+-]?\d+)?$")


def _coerce_number(v):
    """PyYAML (YAML 1.1) reads ``1e-6`` as a string; turn such strings into numbers."""
    if isinstance(v, str) and _NUM.match(v.strip()):
        f = float(v)
        return int(f) if re.fullmatch(r"[+-]?\d+", v.strip()) else f
    return v


def _coerce_tree(node):
    if isinstance(node, dict):
        for k in list(node.keys()):
            v = node[k]
            if isinstance(v, (dict, list)):
                _coerce_tree(v)
            else:
                r = _coerce_number(v)
                if r is not v:
                    dict.__setitem__(node, k, r)
    elif isinstance(node, list):
        for i, v in enumerate(node):
            if isinstance(v, (dict, list)):
                _coerce_tree(v)
            else:
                node[i] = _coerce_number(v)
    return node


def _parse_scalar(text: str):
    try:
        return _coerce_number(yaml.safe_load(text))
    except Exception:
        return text


def _merge(dst: dict, src: dict) -> dict:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _merge(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v)
    return dst


def compose(config_dir: str, config_name: str, group_choices: Optional[dict] = None) -> dict:
    """Load ``config_name`` from ``config_dir`` resolving its ``defaults:`` list recursively."""
    group_choices = group_choices or {}
    path = os.path.join(config_dir, config_name if config_name.endswith(".yaml") else config_name + ".yaml")
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    defaults = raw.pop("defaults", None) or []
    out: dict = {}
    self_done = False
    for item in defaults:
        if item == "_self_":
            _merge(out, raw)
            self_done = True
            continue
        if isinstance(item, str):
            _merge(out, compose(os.path.dirname(os.path.join(config_dir, item)) or config_dir,
                                os.path.basename(item), group_choices))
            continue
        (key, option), = item.items()
        if option is None or option == "null":
            continue
        key = key.replace("optional ", "").replace("override ", "").strip()
        group, _, target = key.partition("@")
        option = group_choices.get(key, group_choices.get(group, option))
        sub = compose(os.path.join(config_dir, group), str(option), group_choices)
        target = target or group.replace("/", ".")
        node = out
        parts = target.split(".")
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        if isinstance(node.get(parts[-1]), dict):
            _merge(node[parts[-1]], sub)
        else:
            node[parts[-1]] = sub
    if not self_done:
        _merge(out, raw)
    return out


_INTERP = re.compile(r"\$\{([^${}]+)\}")


def _resolve(root: DictConfig, value, depth: int = 0, parent=None):
    if depth > 20 or not isinstance(value, str) or "${" not in value:
        return value

    def lookup(expr: str):
        expr = expr.strip()
        if expr.startswith(".") and parent is not None:
            cur = parent
            for part in expr.lstrip(".").split("."):
                cur = cur.get(part) if isinstance(cur, dict) else None
            return cur
        if expr.startswith("oc.select:"):
            key, _, default = expr[len("oc.select:"):].partition(",")
            got = root.select(key.strip(), None)
            return got if got is not None else _parse_scalar(default.strip())
        if expr.startswith("oc.env:"):
            key, _, default = expr[len("oc.env:"):].partition(",")
            return os.environ.get(key.strip(), _parse_scalar(default.strip()) if default else None)
        return root.select(expr, None)

    m = _INTERP.fullmatch(value)
    if m:
        return _resolve(root, lookup(m.group(1)), depth + 1, parent)
    return _resolve(root, _INTERP.sub(lambda mm: str(lookup(mm.group(1))), value), depth + 1, parent)


def resolve_interpolations(cfg: DictConfig) -> DictConfig:
    def walk(node):
        if isinstance(node, dict):
            for k in list(node.keys()):
                v = node[k]
                if isinstance(v, (dict, list)):
                    walk(v)
                else:
                    r = _resolve(cfg, v, 0, node)
                    if r is not v:
                        dict.__setitem__(node, k, DictConfig._wrap(r))
        elif isinstance(node, list):
            for i, v in enumerate(node):
                if isinstance(v, (dict, list)):
                    walk(v)
                else:
                    node[i] = _resolve(cfg, v)

    walk(cfg)
    return cfg


def apply_overrides(cfg: DictConfig, overrides: Iterable[str]) -> DictConfig:
    for ov in overrides or []:
        ov = ov.strip()
        if not ov:
            continue
        if ov.startswith("~"):
            path = ov[1:].split("=")[0]
            parent, _, leaf = path.rpartition(".")
            node = cfg.select(parent) if parent else cfg
            if isinstance(node, dict):
                node.pop(leaf, None)
            continue
        key, sep, val = ov.partition("=")
        if not sep:
            raise ValueError(f"override '{ov}' is not of the form key=value")
        key = key.lstrip("+")
        cfg.set_path(key, _parse_scalar(val))
    return cfg


def load_config(config_dir: str, config_name: str, overrides: Optional[Iterable[str]] = None) -> DictConfig:
    overrides = list(overrides or [])
    choices = {}
    rest = []
    for ov in overrides:
        k, sep, v = ov.partition("=")
        group = k.split("@")[0].lstrip("+")  # "actor@actor_rollout_ref.actor=megatron_actor": group "actor" packaged at a path
        if sep and "." not in group and os.path.isdir(os.path.join(config_dir, group)) and \
                os.path.exists(os.path.join(config_dir, group, v + ".yaml")):
            choices[k.lstrip("+")] = v
        else:
            rest.append(ov)
    cfg = DictConfig(_coerce_tree(compose(config_dir, config_name, choices)))
    apply_overrides(cfg, rest)
    return resolve_interpolations(cfg)


def omega_conf_to_dataclass(config, dataclass_type=None):
    """Instantiate the dataclass named by ``_target_`` (or ``dataclass_type``) from a config node."""
    if config is None:
        return None if dataclass_type is None else dataclass_type()
    if is_dataclass(config) and not isinstance(config, type):
        return config
    if dataclass_type is None:
        target = config.get("_target_") if isinstance(config, dict) else None
        if not target:
            return config
        mod, _, name = target.rpartition(".")
        mod = mod.replace("verl.", "verl_b200.", 1) if mod.startswith("verl.") else mod
        dataclass_type = getattr(importlib.import_module(mod), name)
    data = {k: v for k, v in dict(config).items() if k != "_target_"}
    if hasattr(dataclass_type, "from_dict"):
        return dataclass_type.from_dict(data)
    names = {f.name for f in fields(dataclass_type)}
    return dataclass_type(**{k: v for k, v in data.items() if k in names})


def update_dict_with_config(dictionary: dict, config) -> None:
    for k in dictionary:
        if k in config:
            dictionary[k] = config[k]


def validate_config(config, use_reference_policy: bool = False, use_critic: bool = False) -> None:
    """Cross-field checks of a trainer config (batch-size divisibility, mutually exclusive knobs)."""
    n_gpus = config.trainer.n_gpus_per_node * config.trainer.nnodes
    actor = config.actor_rollout_ref.actor
    rollout = config.actor_rollout_ref.rollout
    real_bsz = config.data.train_batch_size * rollout.n
    if not actor.get("use_dynamic_bsz", False):
        mb, mbg = actor.get("ppo_micro_batch_size"), actor.get("ppo_micro_batch_size_per_gpu")
        if mb is None and mbg is None:
            raise ValueError("[actor] Please set at least one of 'actor.ppo_micro_batch_size' or "
                             "'actor.ppo_micro_batch_size_per_gpu' (or enable use_dynamic_bsz).")
        if mb is not None and mbg is not None:
            raise ValueError("[actor] You have set both 'ppo_micro_batch_size' and 'ppo_micro_batch_size_per_gpu'; "
                             "set only the per-gpu one.")
    assert real_bsz % n_gpus == 0, (f"real_train_batch_size ({real_bsz}) must be divisible by total n_gpus ({n_gpus}).")
    mini = actor.get("ppo_mini_batch_size", config.data.train_batch_size)
    assert config.data.train_batch_size >= mini, "train_batch_size must be >= ppo_mini_batch_size"
    if actor.get("loss_agg_mode", "token-mean") not in ("token-mean", "token-sum", "seq-mean-token-sum",
                                                         "seq-mean-token-mean", "seq-mean-token-sum-norm"):
        raise ValueError(f"Invalid loss_agg_mode: {actor.loss_agg_mode}")
    if config.algorithm.get("use_kl_in_reward", False) and actor.get("use_kl_loss", False):
        print("NOTICE: You have both enabled in-reward kl and kl loss.")
    if use_critic and not config.critic.get("use_dynamic_bsz", False):
        if config.critic.get("ppo_micro_batch_size") is None and config.critic.get("ppo_micro_batch_size_per_gpu") is None:
            raise ValueError("[critic] set ppo_micro_batch_size_per_gpu or enable use_dynamic_bsz")
    if rollout.get("n", 1) > 1 and rollout.get("temperature", 1.0) == 0:
        raise ValueError("rollout.n > 1 requires temperature > 0 (sampling)")
