"""Check that a merged model directory is a complete Hugging Face model before anyone relies on it.

A merge that was interrupted, ran out of disk or wrote an index pointing at shards that never arrived looks fine until the
model is loaded somewhere else. ``validate_hf_model_output`` collects every problem it finds and raises once:

* ``config.json`` exists, is not empty and holds a JSON object;
* weights are present either as one file (``model.safetensors`` / ``pytorch_model.bin``) or as an index whose
  ``weight_map`` is non-empty and whose shard names are plain relative paths inside the directory (no absolute path, no
  ``..``) that exist and are not empty;
* every ``.safetensors`` file named that way has a readable header, and with an index every tensor the index lists is
  in the shard it is listed under.

Parity target: ``verl/model_merger/output_validation.py:34-94`` (the header check goes beyond it).
"""

from __future__ import annotations

import json
import struct
from pathlib import Path, PurePosixPath
from typing import Optional, Union

__all__ = ["validate_hf_model_output", "read_safetensors_names"]

CONFIG_NAME = "config.json"
WEIGHT_NAMES = ("model.safetensors", "pytorch_model.bin")
WEIGHT_INDEX_NAMES = ("model.safetensors.index.json", "pytorch_model.bin.index.json")


def _nonempty(path: Path) -> bool:
    return path.is_file() and path.stat().st_size > 0


def _inside(root: Path, name: str) -> Optional[Path]:
    p = PurePosixPath(name)
    if p.is_absolute() or not p.parts or ".." in p.parts:
        return None
    return root.joinpath(*p.parts)


def read_safetensors_names(path: Union[str, Path]) -> set:
    """Tensor names of a ``.safetensors`` file from its header alone (8-byte little-endian length, then JSON)."""
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError("file shorter than its length prefix")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or n > (100 << 20):
            raise ValueError(f"implausible header length {n}")
        raw = f.read(n)
        if len(raw) != n:
            raise ValueError("truncated header")
    meta = json.loads(raw.decode("utf-8"))
    if not isinstance(meta, dict):
        raise ValueError("header is not a JSON object")
    return {k for k in meta if k != "__metadata__"}


def validate_hf_model_output(target_dir: Union[str, Path]) -> None:
    root = Path(target_dir)
    errors: list[str] = []
    cfg = root / CONFIG_NAME
    if not _nonempty(cfg):
        errors.append(f"missing or empty {CONFIG_NAME}")
    else:
        try:
            if not isinstance(json.loads(cfg.read_text(encoding="utf-8")), dict):
                errors.append(f"{CONFIG_NAME} must contain a JSON object")
        except (OSError, UnicodeError, json.JSONDecodeError) as e:
            errors.append(f"invalid {CONFIG_NAME}: {e}")

    complete = False
    for name in WEIGHT_NAMES:
        if _nonempty(root / name):
            if name.endswith(".safetensors"):
                try:
                    read_safetensors_names(root / name)
                except (OSError, ValueError, UnicodeError, json.JSONDecodeError) as e:
                    errors.append(f"unreadable {name}: {e}")
                    continue
            complete = True
    index_errors: list[str] = []
    for index_name in WEIGHT_INDEX_NAMES:
        ip = root / index_name
        if not ip.exists():
            continue
        try:
            index = json.loads(ip.read_text(encoding="utf-8"))
        except (OSError, UnicodeError, json.JSONDecodeError) as e:
            index_errors.append(f"invalid {index_name}: {e}")
            continue
        wm = index.get("weight_map") if isinstance(index, dict) else None
        if not isinstance(wm, dict) or not wm:
            index_errors.append(f"{index_name} has no non-empty weight_map")
            continue
        if not all(isinstance(v, str) and v for v in wm.values()):
            index_errors.append(f"{index_name} contains invalid shard names")
            continue
        paths = {s: _inside(root, s) for s in set(wm.values())}
        unsafe = sorted(s for s, p in paths.items() if p is None)
        if unsafe:
            index_errors.append(f"{index_name} contains unsafe shard paths: {unsafe}")
            continue
        missing = sorted(s for s, p in paths.items() if not _nonempty(p))
        if missing:
            index_errors.append(f"{index_name} references missing or empty shards: {missing}")
            continue
        bad = []
        for s, p in sorted(paths.items()):
            if not s.endswith(".safetensors"):
                continue
            try:
                have = read_safetensors_names(p)
            except (OSError, ValueError, UnicodeError, json.JSONDecodeError) as e:
                bad.append(f"{s}: {e}")
                continue
            lost = sorted(k for k, v in wm.items() if v == s and k not in have)
            if lost:
                bad.append(f"{s} lacks {len(lost)} tensors the index lists under it (first: {lost[0]})")
        if bad:
            index_errors.append(f"{index_name} does not match its shards: {bad}")
            continue
        complete = True
    if not complete:
        errors += index_errors
        errors.append("no complete model weights; expected one of: " + ", ".join((*WEIGHT_NAMES, *WEIGHT_INDEX_NAMES)))
    if errors:
        raise RuntimeError(f"Incomplete Hugging Face model output at {root}: " + "; ".join(errors))
