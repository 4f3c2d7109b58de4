"""Data protocol of the single-controller runtime.

``DataProto`` is the unit exchanged between the driver and worker groups: a batch-first
:class:`TensorDict` (``batch``), a dict of per-row numpy object arrays (``non_tensor_batch``) and a free
form ``meta_info`` dict that applies to the whole batch.  The driver splits it along the batch
dimension for dispatch and concatenates the per-rank results on collect.

Behavioural parity target: ``verl/protocol.py`` (``DataProto`` :317-1170, ``DataProtoFuture`` :1173,
``pad_dataproto_to_divisor`` :74, ``unpad_dataproto`` :102, ``union_tensor_dict`` :109,
``all_gather_data_proto`` :1334).
"""

from __future__ import annotations

import contextlib
import copy
import io
import os
import pickle
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator, Optional, Sequence

import numpy as np
import torch

from .utils.tensordict_lite import NestedRows, NonTensor, TensorDict, cat_tensordicts

__all__ = [
    "DataProto",
    "DataProtoItem",
    "DataProtoFuture",
    "DataProtoConfig",
    "BatchData",
    "union_tensor_dict",
    "union_numpy_dict",
    "pad_dataproto_to_divisor",
    "unpad_dataproto",
    "fold_batch_dim",
    "unfold_batch_dim",
    "collate_fn",
    "list_of_dict_to_dict_of_list",
    "all_gather_data_proto",
]


class _AutoPaddingConfig:
    """Process-wide switch for transparent padding on chunk (env ``VERL_AUTO_PADDING``)."""

    auto_padding_key = "_verl_auto_padding"

    @property
    def auto_padding(self) -> bool:
        return os.getenv("VERL_AUTO_PADDING", "FALSE").upper() in ("TRUE", "1")


DataProtoConfig = _AutoPaddingConfig()


def pad_dataproto_to_divisor(data: "DataProto", size_divisor: int):
    """Pad by cycling the batch's own rows until ``len % size_divisor == 0``. Returns (padded, pad)."""
    assert isinstance(data, DataProto), "data must be a DataProto"
    n = len(data)
    if n % size_divisor == 0 or n == 0:
        return data, 0
    pad = size_divisor - n % size_divisor
    pieces = [data]
    remaining = pad
    while remaining > 0:
        take = min(remaining, n)
        pieces.append(data[:take])
        remaining -= take
    return DataProto.concat(pieces), pad


def unpad_dataproto(data: "DataProto", pad_size: int) -> "DataProto":
    return data[:-pad_size] if pad_size else data


def union_tensor_dict(a: TensorDict, b: TensorDict) -> TensorDict:
    """Merge ``b`` into ``a``; keys present in both must hold equal tensors."""
    assert a.batch_size == b.batch_size, f"batch size mismatch {a.batch_size} vs {b.batch_size}"
    for k in b.keys():
        vb = b._data[k]
        if k in a:
            va = a._data[k]
            if isinstance(va, NonTensor) or isinstance(vb, NonTensor):
                same = isinstance(va, NonTensor) and isinstance(vb, NonTensor) and _obj_equal(va.data, vb.data)
            elif isinstance(va, NestedRows) or isinstance(vb, NestedRows):
                same = (isinstance(va, NestedRows) and isinstance(vb, NestedRows)
                        and torch.equal(va.offsets, vb.offsets) and torch.equal(va.values, vb.values))
            else:
                same = va.shape == vb.shape and torch.equal(va, vb.to(va.device))
            assert same, f"'{k}' differs between the two batches"
        else:
            a._data[k] = vb
    return a


def _obj_equal(x, y) -> bool:
    try:
        r = x == y
        if isinstance(r, (np.ndarray, torch.Tensor)):
            return bool(r.all())
        return bool(r)
    except Exception:
        return False


def _np_rows_equal(x: np.ndarray, y: np.ndarray) -> bool:
    if x.shape != y.shape:
        return False
    if x.dtype != object and y.dtype != object:
        return bool(np.array_equal(x, y, equal_nan=np.issubdtype(x.dtype, np.floating)))
    for xi, yi in zip(x.reshape(-1), y.reshape(-1)):
        if isinstance(xi, float) and isinstance(yi, float) and np.isnan(xi) and np.isnan(yi):
            continue
        if not _obj_equal(xi, yi):
            return False
    return True


def union_numpy_dict(a: dict[str, np.ndarray], b: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    for k, v in b.items():
        if k in a:
            assert isinstance(v, np.ndarray) and isinstance(a[k], np.ndarray)
            assert _np_rows_equal(a[k], v), f"'{k}' differs between the two non-tensor batches"
        a[k] = v
    return a


def list_of_dict_to_dict_of_list(items: Sequence[dict]) -> dict[str, list]:
    if not items:
        return {}
    keys = items[0].keys()
    out = {k: [] for k in keys}
    for it in items:
        assert it.keys() == keys
        for k, v in it.items():
            out[k].append(v)
    return out


def fold_batch_dim(data: "DataProto", new_batch_size: int) -> "DataProto":
    """[bsz, ...] -> [new_batch_size, bsz // new_batch_size, ...] on every entry."""
    n = len(data)
    assert n % new_batch_size == 0
    td = TensorDict({k: v.reshape(new_batch_size, -1, *v.shape[1:]) for k, v in data.batch.items()
                     if isinstance(v, torch.Tensor)}, batch_size=(new_batch_size,))
    non = {k: v.reshape(new_batch_size, -1, *v.shape[1:]) for k, v in data.non_tensor_batch.items()}
    return DataProto(batch=td, non_tensor_batch=non, meta_info=data.meta_info)


def unfold_batch_dim(data: "DataProto", batch_dims: int = 2) -> "DataProto":
    """Inverse of :func:`fold_batch_dim`: merge the first ``batch_dims`` dims."""
    td = TensorDict({k: v.reshape(-1, *v.shape[batch_dims:]) for k, v in data.batch.items()
                     if isinstance(v, torch.Tensor)})
    bsz = len(td)
    non = {k: v.reshape(bsz, *v.shape[batch_dims:]) for k, v in data.non_tensor_batch.items()}
    return DataProto(batch=td, non_tensor_batch=non, meta_info=data.meta_info)


def collate_fn(items: Sequence["DataProtoItem"]) -> "DataProto":
    tensors = [it.batch for it in items]
    non = list_of_dict_to_dict_of_list([it.non_tensor_batch for it in items])
    batch = {k: torch.stack([t[k] for t in tensors]) for k in (tensors[0].keys() if tensors[0] else [])}
    return DataProto.from_dict(tensors=batch, non_tensors={k: _to_object_array(v) for k, v in non.items()})


def _to_object_array(values) -> np.ndarray:
    if isinstance(values, np.ndarray):
        return values
    arr = np.empty(len(values), dtype=object)
    for i, v in enumerate(values):
        arr[i] = v
    return arr


@dataclass
class DataProtoItem:
    batch: Optional[dict] = None
    non_tensor_batch: dict = field(default_factory=dict)
    meta_info: dict = field(default_factory=dict)


@dataclass
class DataProto:
    batch: Optional[TensorDict] = None
    non_tensor_batch: dict = field(default_factory=dict)
    meta_info: dict = field(default_factory=dict)

    def __post_init__(self):
        self.check_consistency()

    # ------------------------------------------------------------------------------- sizes
    def __len__(self) -> int:
        if self.batch is not None and len(self.batch.tensor_keys()):
            return self.batch.batch_size[0]
        if self.batch is not None and self.batch.batch_size and not self.non_tensor_batch:
            return self.batch.batch_size[0]
        if self.non_tensor_batch:
            return next(iter(self.non_tensor_batch.values())).shape[0]
        return 0

    def __getitem__(self, item):
        if isinstance(item, slice):
            return self.slice(item.start, item.stop, item.step)
        if isinstance(item, (list, np.ndarray, torch.Tensor)):
            return self.select_idxs(item)
        if isinstance(item, (int, np.integer)):
            i = int(item)
            td = {k: (v.row(i) if isinstance(v, NestedRows) else v[i]) for k, v in self.batch.items()
                  if not isinstance(v, NonTensor)} if self.batch is not None else None
            non = {k: v[i] for k, v in self.non_tensor_batch.items()}
            return DataProtoItem(batch=td, non_tensor_batch=non, meta_info=self.meta_info)
        raise TypeError(f"unsupported index type {type(item)}")

    # ------------------------------------------------------------------------------- pickling
    def __getstate__(self):
        method = os.getenv("VERL_DATAPROTO_SERIALIZATION_METHOD", "torch")
        batch = self.batch.contiguous() if self.batch is not None else None
        if method == "numpy" and batch is not None:
            enc = {}
            for k, v in batch.items():
                if isinstance(v, torch.Tensor):
                    t = v.detach().cpu()
                    enc[k] = ("t", str(t.dtype), t.view(torch.uint8).numpy() if t.dtype == torch.bfloat16
                              else t.numpy(), tuple(t.shape))
                else:
                    enc[k] = ("o", v)
            return {"mode": "numpy", "batch": enc, "bsz": tuple(batch.batch_size),
                    "non": self.non_tensor_batch, "meta": self.meta_info}
        buf = io.BytesIO()
        torch.save(batch, buf)
        return {"mode": "torch", "batch": buf.getvalue(), "non": self.non_tensor_batch, "meta": self.meta_info}

    def __setstate__(self, state):
        if state["mode"] == "numpy":
            src = {}
            for k, e in state["batch"].items():
                if e[0] == "t":
                    dt = getattr(torch, e[1].split(".")[-1])
                    t = torch.from_numpy(np.ascontiguousarray(e[2]))
                    src[k] = t.view(dt).reshape(e[3]) if dt == torch.bfloat16 else t
                else:
                    src[k] = e[1]
            self.batch = TensorDict(src, batch_size=state["bsz"])
        else:
            self.batch = torch.load(io.BytesIO(state["batch"]), weights_only=False,
                                    map_location="cpu" if not torch.cuda.is_available() else None)
        self.non_tensor_batch = state["non"]
        self.meta_info = state["meta"]

    def save_to_disk(self, filepath: str) -> None:
        with open(filepath, "wb") as f:
            pickle.dump(self, f)

    @staticmethod
    def load_from_disk(filepath: str) -> "DataProto":
        with open(filepath, "rb") as f:
            return pickle.load(f)

    def print_size(self, prefix: str = "") -> None:
        tb = 0
        if self.batch is not None:
            for v in self.batch.values():
                if isinstance(v, torch.Tensor):
                    tb += v.element_size() * v.numel()
                elif isinstance(v, NestedRows):
                    tb += v.values.element_size() * v.values.numel()
        nb = sum(v.nbytes for v in self.non_tensor_batch.values())
        msg = f"Size of tensordict: {tb / 1024**3:.4f} GB, size of non_tensor_batch: {nb / 1024**3:.4f} GB"
        print(f"{prefix}, {msg}" if prefix else msg)

    # ------------------------------------------------------------------------------- invariants
    def check_consistency(self) -> None:
        if self.batch is not None:
            assert len(self.batch.batch_size) == 1, "only one batch dimension is supported"
        for k, v in self.non_tensor_batch.items():
            assert isinstance(v, np.ndarray), f"non_tensor_batch['{k}'] must be a numpy array, got {type(v)}"
        if self.batch is not None and self.non_tensor_batch and len(self.batch.tensor_keys()):
            bsz = self.batch.batch_size[0]
            for k, v in self.non_tensor_batch.items():
                assert v.shape[0] == bsz, f"non-tensor '{k}' has {v.shape[0]} rows, batch has {bsz}"

    # ------------------------------------------------------------------------------- constructors
    @classmethod
    def from_single_dict(cls, data: dict[str, Any], meta_info: dict | None = None, auto_padding: bool = False):
        tensors, non = {}, {}
        for k, v in data.items():
            if isinstance(v, (torch.Tensor, NestedRows)):
                tensors[k] = v
            elif isinstance(v, np.ndarray):
                non[k] = v
            else:
                raise ValueError(f"unsupported value type {type(v)} for key '{k}'")
        return cls.from_dict(tensors=tensors, non_tensors=non, meta_info=meta_info, auto_padding=auto_padding)

    @classmethod
    def from_dict(cls, tensors: dict | None = None, non_tensors: dict | None = None, meta_info: dict | None = None,
                  num_batch_dims: int = 1, auto_padding: bool = False):
        assert num_batch_dims > 0
        tensors = tensors or {}
        non_tensors = non_tensors or {}
        meta_info = dict(meta_info or {})
        assert isinstance(non_tensors, dict)
        bdims, pivot = None, None
        for k, t in tensors.items():
            cur = (len(t),) if isinstance(t, NestedRows) else tuple(t.shape[:num_batch_dims])
            if bdims is None:
                bdims, pivot = cur, k
            else:
                assert cur == bdims, f"batch dims of '{k}' {cur} differ from '{pivot}' {bdims}"
        non = {k: _to_object_array(v) if not isinstance(v, np.ndarray) else v for k, v in non_tensors.items()}
        td = TensorDict(tensors, batch_size=bdims) if tensors else None
        if auto_padding:
            meta_info[DataProtoConfig.auto_padding_key] = True
        return cls(batch=td, non_tensor_batch=non, meta_info=meta_info)

    @classmethod
    def from_tensordict(cls, tensor_dict: TensorDict, meta_info: dict | None = None, num_batch_dims: int = 1):
        tensors, non, meta = {}, {}, dict(meta_info or {})
        n = len(tensor_dict)
        for k, v in tensor_dict.items():
            if isinstance(v, NonTensor):
                d = v.data
                if isinstance(d, np.ndarray) and d.ndim >= 1 and d.shape[0] == n:
                    non[k] = d
                elif isinstance(d, (list, tuple)) and len(d) == n:
                    non[k] = _to_object_array(list(d))
                else:
                    meta[k] = d
            else:
                tensors[k] = v
        return cls.from_dict(tensors=tensors, non_tensors=non, meta_info=meta, num_batch_dims=num_batch_dims)

    def to_tensordict(self) -> TensorDict:
        """One TensorDict carrying tensors, per-row non-tensors (as lists) and meta_info (as non-tensors)."""
        src: dict[str, Any] = {}
        if self.batch is not None:
            src.update(self.batch._data)
        for k, v in self.non_tensor_batch.items():
            src[k] = NonTensor(v)
        for k, v in self.meta_info.items():
            src[k] = NonTensor(v)
        return TensorDict(src, batch_size=(len(self),))

    # ------------------------------------------------------------------------------- device / select
    def to(self, device) -> "DataProto":
        if self.batch is not None:
            self.batch = self.batch.to(device)
        return self

    def select(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None, deepcopy: bool = False):
        td = self.batch
        if batch_keys is not None and td is not None:
            td = td.select(*tuple(batch_keys))
        non = self.non_tensor_batch
        if non_tensor_batch_keys is not None:
            non = {k: v for k, v in non.items() if k in non_tensor_batch_keys}
        meta = self.meta_info
        if meta_info_keys is not None:
            meta = {k: v for k, v in meta.items() if k in meta_info_keys}
        if deepcopy:
            non, meta = copy.deepcopy(non), copy.deepcopy(meta)
        return type(self)(batch=td, non_tensor_batch=dict(non), meta_info=dict(meta))

    def select_idxs(self, idxs) -> "DataProto":
        if isinstance(idxs, list):
            idxs = torch.tensor(idxs, dtype=torch.bool if idxs and isinstance(idxs[0], bool) else torch.int64)
        if isinstance(idxs, np.ndarray):
            np_idx, t_idx = idxs, torch.from_numpy(idxs)
        else:
            t_idx, np_idx = idxs, idxs.detach().cpu().numpy()
        td = self.batch[t_idx] if self.batch is not None else None
        non = {k: v[np_idx] for k, v in self.non_tensor_batch.items()}
        return type(self)(batch=td, non_tensor_batch=non, meta_info=self.meta_info)

    def slice(self, start=None, end=None, step=None) -> "DataProto":
        sl = slice(start, end, step)
        td = self.batch[sl] if self.batch is not None else None
        non = {k: v[sl] for k, v in self.non_tensor_batch.items()}
        return type(self)(batch=td, non_tensor_batch=non, meta_info=self.meta_info)

    def pop(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None) -> "DataProto":
        batch_keys = batch_keys or []
        non_tensor_batch_keys = non_tensor_batch_keys or []
        meta_info_keys = meta_info_keys or []
        tensors = {k: self.batch.pop(k) for k in batch_keys}
        non = {k: self.non_tensor_batch.pop(k) for k in non_tensor_batch_keys}
        meta = {k: self.meta_info.pop(k) for k in meta_info_keys}
        return DataProto.from_dict(tensors=tensors, non_tensors=non, meta_info=meta)

    def rename(self, old_keys=None, new_keys=None) -> "DataProto":
        def as_list(k):
            if k is None:
                return []
            if isinstance(k, str):
                return [k]
            if isinstance(k, list):
                return k
            raise TypeError(f"keys must be str or list, got {type(k)}")

        old_keys, new_keys = as_list(old_keys), as_list(new_keys)
        if len(old_keys) != len(new_keys):
            raise ValueError(f"{len(old_keys)} old keys vs {len(new_keys)} new keys")
        for o, n in zip(old_keys, new_keys):
            self.batch.rename_key_(o, n)
        return self

    def union(self, other: "DataProto") -> "DataProto":
        if self.batch is None:
            self.batch = other.batch
        elif other.batch is not None:
            self.batch = union_tensor_dict(self.batch, other.batch)
        self.non_tensor_batch = union_numpy_dict(self.non_tensor_batch, other.non_tensor_batch)
        for k, v in other.meta_info.items():
            if k in self.meta_info and not _obj_equal(self.meta_info[k], v) and k != "metrics":
                raise AssertionError(f"meta_info['{k}'] conflicts in union")
            self.meta_info[k] = v
        return self

    # ------------------------------------------------------------------------------- iteration
    def make_iterator(self, mini_batch_size: int, epochs: int, seed=None, dataloader_kwargs=None) -> Iterator["DataProto"]:
        n = len(self)
        assert n % mini_batch_size == 0, f"{n} % {mini_batch_size} != 0"
        dataloader_kwargs = dataloader_kwargs or {}
        shuffle = dataloader_kwargs.get("shuffle", True)
        gen = torch.Generator()
        if seed is not None:
            gen.manual_seed(int(seed))
        for _ in range(epochs):
            order = torch.randperm(n, generator=gen) if shuffle else torch.arange(n)
            for s in range(0, n, mini_batch_size):
                part = self.select_idxs(order[s : s + mini_batch_size])
                part.meta_info = self.meta_info
                yield part

    # ------------------------------------------------------------------------------- padding
    def is_padding_enabled(self) -> bool:
        return bool(self.meta_info.get(DataProtoConfig.auto_padding_key, False)) or DataProtoConfig.auto_padding

    def padding(self, padding_size: int, padding_candidate: str = "") -> None:
        if padding_size == 0:
            return
        cand = self.select_idxs([0 if padding_candidate == "first" else len(self) - 1])
        merged = DataProto.concat([self] + [cand] * padding_size)
        self.batch, self.non_tensor_batch = merged.batch, merged.non_tensor_batch

    # ------------------------------------------------------------------------------- split / merge
    def chunk(self, chunks: int) -> list["DataProto"]:
        n = len(self)
        if not self.is_padding_enabled():
            assert n % chunks == 0, f"only equal chunks are supported: {n} rows into {chunks} chunks"
            size = n // chunks
            return [self.slice(i * size, (i + 1) * size) for i in range(chunks)]
        size = (n + chunks - 1) // chunks
        return [self.slice(i * size, min((i + 1) * size, n)) for i in range(chunks)]

    def split(self, split_size: int) -> list["DataProto"]:
        return [self[i : i + split_size] for i in range(0, len(self), split_size)]

    @staticmethod
    def concat(data: Sequence["DataProto"]) -> "DataProto":
        data = list(data)
        assert len(data) > 0
        tds = [d.batch for d in data if d.batch is not None]
        td = cat_tensordicts(tds) if tds else None
        non_keys = data[0].non_tensor_batch.keys()
        non = {k: np.concatenate([d.non_tensor_batch[k] for d in data], axis=0) for k in non_keys}
        # meta_info: 'metrics' lists/dicts are aggregated, every other key must agree.
        merged: dict[str, Any] = {}
        metric_items = []
        for d in data:
            for k, v in d.meta_info.items():
                if k == "metrics":
                    if v is not None:
                        metric_items.extend(v if isinstance(v, list) else [v])
                elif k in merged:
                    assert _obj_equal(merged[k], v), f"conflicting meta_info['{k}'] in concat"
                else:
                    merged[k] = v
        if metric_items:
            merged["metrics"] = list_of_dict_to_dict_of_list(metric_items)
        cls = type(data[0])
        return cls(batch=td, non_tensor_batch=non, meta_info=merged)

    def reorder(self, indices: torch.Tensor) -> None:
        self.batch = self.batch[indices]
        np_idx = indices.detach().cpu().numpy()
        self.non_tensor_batch = {k: v[np_idx] for k, v in self.non_tensor_batch.items()}

    def repeat(self, repeat_times: int = 2, interleave: bool = True) -> "DataProto":
        n = len(self)
        idx = (torch.arange(n).repeat_interleave(repeat_times) if interleave
               else torch.arange(n).repeat(repeat_times))
        out = self.select_idxs(idx)
        out.meta_info = self.meta_info
        return out

    def sample_level_repeat(self, repeat_times) -> "DataProto":
        if isinstance(repeat_times, (tuple, list)):
            reps = torch.tensor(repeat_times)
        elif isinstance(repeat_times, np.ndarray):
            reps = torch.from_numpy(repeat_times)
        else:
            reps = repeat_times
        assert reps.dim() == 1 and reps.numel() == len(self)
        idx = torch.arange(len(self)).repeat_interleave(reps.to(torch.int64))
        return self.select_idxs(idx)

    def unfold_column_chunks(self, n_split: int, split_keys: Sequence[str] | None = None) -> "DataProto":
        """Split dim 1 of ``split_keys`` into ``n_split`` pieces moved to the batch dim; other keys repeat."""
        split_keys = list(split_keys or [])
        tensors = {}
        for k, v in self.batch.items():
            if not isinstance(v, torch.Tensor):
                continue
            if k in split_keys:
                shape = list(v.shape)
                tensors[k] = v.reshape(shape[0] * n_split, shape[1] // n_split, *shape[2:])
            else:
                tensors[k] = v.repeat_interleave(n_split, dim=0)
        non = {}
        for k, v in self.non_tensor_batch.items():
            if k in split_keys:
                shape = list(v.shape)
                non[k] = v.reshape(shape[0] * n_split, shape[1] // n_split, *shape[2:])
            else:
                non[k] = np.repeat(v, n_split, axis=0)
        return type(self).from_dict(tensors=tensors, non_tensors=non, meta_info=self.meta_info)

    def get_data_info(self) -> str:
        lines = ["batch"]
        if self.batch is not None:
            for k, v in self.batch.items():
                if isinstance(v, torch.Tensor):
                    lines.append(f"  {k}: {tuple(v.shape)} ({v.dtype}) {v.device}")
                else:
                    lines.append(f"  {k}: {v!r}")
        lines.append("non_tensor_batch")
        for k, v in self.non_tensor_batch.items():
            lines.append(f"  {k}: ndarray{v.shape} ({v.dtype})")
        lines.append("meta_info")
        for k, v in self.meta_info.items():
            lines.append(f"  {k}: {type(v).__name__}")
        return "\n".join(lines)


# ---------------------------------------------------------------------------------------------------
@dataclass
class DataProtoFuture:
    """Lazy result of an asynchronous worker-group call.

    ``futures`` is a list of objects with ``.result()`` (``concurrent.futures``) or plain values;
    ``collect_fn`` merges the per-worker outputs into one DataProto and ``dispatch_fn`` (set by
    :meth:`chunk`) picks this consumer's slice, so a future can be forwarded to another worker group
    without materialising it on the driver first.
    """

    collect_fn: Callable
    futures: list
    dispatch_fn: Optional[Callable] = None

    @staticmethod
    def concat(data: list) -> "DataProtoFuture":
        return DataProtoFuture(collect_fn=DataProto.concat, futures=list(data))

    def chunk(self, chunks: int) -> list["DataProtoFuture"]:
        from functools import partial

        def pick(x, i, chunks):
            return x.chunk(chunks=chunks)[i]

        return [DataProtoFuture(collect_fn=self.collect_fn, futures=self.futures,
                                dispatch_fn=partial(pick, i=i, chunks=chunks)) for i in range(chunks)]

    def get(self):
        outs = [f.result() if hasattr(f, "result") else f for f in self.futures]
        for o in outs:
            assert isinstance(o, DataProto)
        out = self.collect_fn(outs)
        return self.dispatch_fn(out) if self.dispatch_fn is not None else out


class BatchData:
    """Uniform chunk/concat over the batch carriers the trainers pass around."""

    @staticmethod
    def chunk(data, chunks: int):
        if isinstance(data, (DataProto, DataProtoFuture)):
            return data.chunk(chunks)
        if isinstance(data, TensorDict):
            from .utils.tensordict_lite import chunk_tensordict

            return chunk_tensordict(data, chunks)
        raise TypeError(f"cannot chunk {type(data)}")

    @staticmethod
    def concat(items: Sequence):
        first = items[0]
        if isinstance(first, DataProto):
            return DataProto.concat(items)
        if isinstance(first, DataProtoFuture):
            return DataProtoFuture.concat(items)
        if isinstance(first, TensorDict):
            return cat_tensordicts(items)
        raise TypeError(f"cannot concat {type(first)}")

    @staticmethod
    def length(data) -> int:
        return len(data)


def all_gather_data_proto(data: DataProto, process_group=None) -> None:
    """In-place all-gather of a DataProto across ``process_group`` (object collective)."""
    import torch.distributed as dist

    world = dist.get_world_size(group=process_group)
    gathered: list = [None] * world
    dev = data.batch.device if data.batch is not None else None
    dist.all_gather_object(gathered, data.to("cpu") if dev is not None else data, group=process_group)
    merged = DataProto.concat(gathered)
    data.batch = merged.batch.to(dev) if (merged.batch is not None and dev is not None) else merged.batch
    data.non_tensor_batch = merged.non_tensor_batch
