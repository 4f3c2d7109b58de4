"""Typed configuration base: frozen, mapping-like dataclasses with an allow-list of mutable fields.

Parity target: ``verl/base_config.py:21-86``.
"""

from __future__ import annotations

import collections.abc
from dataclasses import FrozenInstanceError, dataclass, fields, is_dataclass
from typing import Any

__all__ = ["BaseConfig"]


@dataclass
class BaseConfig(collections.abc.Mapping):
    """Dataclass that also behaves like a read-only dict.

    Fields named in ``_mutable_fields`` may be re-assigned after construction; any other assignment to an
    already-set field raises ``FrozenInstanceError``.  Unknown keys given to :meth:`from_dict` are kept in
    ``extra`` when the subclass declares that field.
    """

    _mutable_fields = set()
    _target_: str = ""

    def __setattr__(self, name: str, value):
        if name in self.__dict__ and name not in getattr(self, "_mutable_fields", set()):
            raise FrozenInstanceError(f"Field '{name}' is frozen and cannot be modified")
        super().__setattr__(name, value)

    def get(self, key: str, default: Any = None) -> Any:
        v = getattr(self, key, default)
        return v

    def __getitem__(self, key: str):
        try:
            return getattr(self, key)
        except AttributeError:
            raise KeyError(key) from None

    def __iter__(self):
        for f in fields(self):
            yield f.name

    def __len__(self):
        return len(fields(self))

    def __contains__(self, key) -> bool:
        return any(f.name == key for f in fields(self))

    def to_dict(self) -> dict:
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            out[f.name] = v.to_dict() if isinstance(v, BaseConfig) else v
        return out

    @classmethod
    def from_dict(cls, d):
        """Build from a (possibly nested) mapping; nested dataclass fields are built recursively."""
        if isinstance(d, cls):
            return d
        d = dict(d or {})
        d.pop("_target_", None)
        names = {f.name: f for f in fields(cls)}
        kw, extra = {}, {}
        for k, v in d.items():
            if k in names:
                ft = names[k].type
                sub = _resolve_dataclass(ft, cls)
                if sub is not None and isinstance(v, collections.abc.Mapping) and not isinstance(v, BaseConfig):
                    v = sub.from_dict(v) if hasattr(sub, "from_dict") else sub(**v)
                kw[k] = v
            else:
                extra[k] = v
        if extra and "extra" in names:
            kw["extra"] = {**extra, **dict(kw.get("extra") or {})}
        return cls(**kw)


def _resolve_dataclass(ftype, owner):
    import sys
    import typing

    if isinstance(ftype, str):
        mod = sys.modules.get(owner.__module__)
        name = ftype.replace("Optional[", "").rstrip("]").strip("'\" ")
        cand = getattr(mod, name, None)
        return cand if isinstance(cand, type) and is_dataclass(cand) else None
    if isinstance(ftype, type) and is_dataclass(ftype):
        return ftype
    for a in typing.get_args(ftype) or ():
        if isinstance(a, type) and is_dataclass(a):
            return a
    return None
