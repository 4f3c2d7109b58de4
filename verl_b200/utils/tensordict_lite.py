"""A small batch-first tensor dictionary.

The single-controller data protocol needs a container of tensors that share their leading batch
dimension(s) and can be indexed, sliced, chunked, concatenated, moved between devices and pickled as
one unit.  This module provides exactly that and nothing more, so the framework carries no external
dependency for it.  Entries may be dense tensors, jagged lists wrapped in :class:`NestedRows`, or
arbitrary python objects wrapped in :class:`NonTensor` (kept per-batch, not per-row).

Reference behaviour studied: ``verl/utils/tensordict_utils.py`` (construction with non-tensor data,
jagged "nested" tensors, chunk/concat over jagged entries, ``make_iterator``).
"""

from __future__ import annotations

import copy
from typing import Any, Iterable, Iterator, Mapping, Sequence

import numpy as np
import torch

__all__ = [
    "TensorDict",
    "NestedRows",
    "NonTensor",
    "cat_tensordicts",
    "make_iterator",
    "get_tensordict",
    "assign_non_tensor",
    "get_non_tensor_data",
    "index_select_tensor_dict",
    "chunk_tensordict",
    "concat_tensordict",
    "pad_to_divisor",
    "unpad",
]


class NonTensor:
    """Wrapper marking a value that belongs to the batch as a whole (not one per row)."""

    __slots__ = ("data",)

    def __init__(self, data: Any):
        self.data = data

    def __repr__(self) -> str:  # pragma: no cover - cosmetic
        return f"NonTensor({self.data!r})"

    def __eq__(self, other):
        return isinstance(other, NonTensor) and self.data == other.data


class NestedRows:
    """Jagged batch: one 1-D (or k-D with ragged dim 0) tensor per row, stored flat with offsets.

    ``values`` holds the concatenation of all rows along dim 0 and ``offsets`` (int64, length B+1) the
    row boundaries – the packed ``cu_seqlens`` form the attention kernels consume directly.
    """

    def __init__(self, values: torch.Tensor, offsets: torch.Tensor):
        assert offsets.dim() == 1 and offsets.numel() >= 1
        self.values = values
        self.offsets = offsets.to(torch.int64)

    # -- construction -------------------------------------------------------------------------
    @classmethod
    def from_list(cls, rows: Sequence[torch.Tensor]) -> "NestedRows":
        if len(rows) == 0:
            return cls(torch.empty(0), torch.zeros(1, dtype=torch.int64))
        lens = torch.tensor([int(r.shape[0]) for r in rows], dtype=torch.int64)
        offsets = torch.zeros(len(rows) + 1, dtype=torch.int64)
        offsets[1:] = torch.cumsum(lens, 0)
        return cls(torch.cat(list(rows), dim=0), offsets)

    @classmethod
    def from_padded(cls, padded: torch.Tensor, mask: torch.Tensor) -> "NestedRows":
        """Rows of ``padded`` [B, L, ...] restricted to positions where ``mask`` [B, L] is true."""
        mask = mask.bool()
        lens = mask.sum(-1).to(torch.int64)
        offsets = torch.zeros(mask.shape[0] + 1, dtype=torch.int64)
        offsets[1:] = torch.cumsum(lens.cpu(), 0)
        return cls(padded[mask], offsets)

    # -- views ---------------------------------------------------------------------------------
    def __len__(self) -> int:
        return self.offsets.numel() - 1

    @property
    def device(self):
        return self.values.device

    @property
    def dtype(self):
        return self.values.dtype

    def lengths(self) -> torch.Tensor:
        return self.offsets[1:] - self.offsets[:-1]

    def row(self, i: int) -> torch.Tensor:
        return self.values[int(self.offsets[i]) : int(self.offsets[i + 1])]

    def unbind(self) -> list[torch.Tensor]:
        return [self.row(i) for i in range(len(self))]

    def to(self, *args, **kwargs) -> "NestedRows":
        return NestedRows(self.values.to(*args, **kwargs), self.offsets)

    def clone(self) -> "NestedRows":
        return NestedRows(self.values.clone(), self.offsets.clone())

    def to_padded(self, pad_value=0, max_len: int | None = None, left: bool = False) -> torch.Tensor:
        lens = self.lengths()
        B = len(self)
        L = int(max_len if max_len is not None else (lens.max().item() if B else 0))
        out = self.values.new_full((B, L) + tuple(self.values.shape[1:]), pad_value)
        for i in range(B):
            n = int(lens[i])
            if n == 0:
                continue
            if left:
                out[i, L - n :] = self.row(i)
            else:
                out[i, :n] = self.row(i)
        return out

    def index(self, idx) -> "NestedRows":
        if isinstance(idx, slice):
            idx = list(range(*idx.indices(len(self))))
        elif isinstance(idx, torch.Tensor):
            idx = (idx.nonzero().flatten() if idx.dtype == torch.bool else idx).tolist()
        elif isinstance(idx, np.ndarray):
            idx = (np.nonzero(idx)[0] if idx.dtype == bool else idx).tolist()
        return NestedRows.from_list([self.row(int(i)) for i in idx]) if len(idx) else NestedRows(
            self.values[:0], torch.zeros(1, dtype=torch.int64)
        )

    def __repr__(self) -> str:  # pragma: no cover
        return f"NestedRows(B={len(self)}, total={self.values.shape[0]}, dtype={self.values.dtype})"


def _batch_len(v) -> int:
    if isinstance(v, NestedRows):
        return len(v)
    return int(v.shape[0])


class TensorDict:
    """Dictionary of batch-first tensors with a common ``batch_size``."""

    def __init__(self, source: Mapping[str, Any] | None = None, batch_size: Sequence[int] | int | None = None,
                 device=None):
        self._data: dict[str, Any] = {}
        if isinstance(batch_size, int):
            batch_size = (batch_size,)
        self._batch_size = tuple(batch_size) if batch_size is not None else None
        for k, v in (source or {}).items():
            self[k] = v
        if self._batch_size is None:
            self._batch_size = (0,) if not self._tensor_keys() else (_batch_len(self._data[self._tensor_keys()[0]]),)
        if device is not None:
            moved = self.to(device)
            self._data = moved._data

    # -- basic mapping ---------------------------------------------------------------------------
    def _tensor_keys(self) -> list[str]:
        return [k for k, v in self._data.items() if not isinstance(v, NonTensor)]

    @property
    def batch_size(self) -> torch.Size:
        return torch.Size(self._batch_size)

    @property
    def device(self):
        for k in self._tensor_keys():
            return self._data[k].device
        return None

    def keys(self, include_non_tensor: bool = True):
        return list(self._data.keys()) if include_non_tensor else self._tensor_keys()

    def tensor_keys(self):
        return self._tensor_keys()

    def values(self):
        return self._data.values()

    def items(self):
        return self._data.items()

    def __contains__(self, k) -> bool:
        return k in self._data

    def __len__(self) -> int:
        return self._batch_size[0] if self._batch_size else 0

    def get(self, k, default=None):
        v = self._data.get(k, default)
        return v.data if isinstance(v, NonTensor) else v

    def __setitem__(self, k: str, v: Any) -> None:
        if isinstance(v, (torch.Tensor, NestedRows)):
            if self._batch_size is None:
                self._batch_size = (_batch_len(v),)
            nb = len(self._batch_size)
            shape = (len(v),) if isinstance(v, NestedRows) else tuple(v.shape[:nb])
            if shape != self._batch_size[: len(shape)] or len(shape) < min(nb, 1):
                raise ValueError(f"entry '{k}' has leading shape {shape}, expected {self._batch_size}")
            self._data[k] = v
        elif isinstance(v, NonTensor):
            self._data[k] = v
        else:
            self._data[k] = NonTensor(v)

    def __getitem__(self, idx):
        if isinstance(idx, str):
            v = self._data[idx]
            return v.data if isinstance(v, NonTensor) else v
        return self._index(idx)

    def __delitem__(self, k: str) -> None:
        del self._data[k]

    def pop(self, k, *default):
        if k in self._data:
            v = self._data.pop(k)
            return v.data if isinstance(v, NonTensor) else v
        if default:
            return default[0]
        raise KeyError(k)

    def set(self, k, v):
        self[k] = v
        return self

    def update(self, other: Mapping[str, Any]):
        for k, v in other.items():
            self[k] = v
        return self

    def rename_key_(self, old: str, new: str):
        self._data[new] = self._data.pop(old)
        return self

    # -- indexing ----------------------------------------------------------------------------------
    def _index(self, idx) -> "TensorDict":
        out = TensorDict.__new__(TensorDict)
        out._data = {}
        new_len = None
        for k, v in self._data.items():
            if isinstance(v, NonTensor):
                out._data[k] = v
            elif isinstance(v, NestedRows):
                if isinstance(idx, int):
                    idx_ = [idx]
                    out._data[k] = v.index(idx_)
                else:
                    out._data[k] = v.index(idx)
                new_len = len(out._data[k])
            else:
                if isinstance(idx, (list, np.ndarray)):
                    ii = torch.as_tensor(np.asarray(idx))
                    out._data[k] = v[ii.to(v.device)]
                elif isinstance(idx, torch.Tensor):
                    out._data[k] = v[idx.to(v.device)]
                elif isinstance(idx, int):
                    out._data[k] = v[idx : idx + 1] if idx != -1 else v[-1:]
                else:
                    out._data[k] = v[idx]
                new_len = out._data[k].shape[0]
        if new_len is None:
            if isinstance(idx, slice):
                new_len = len(range(*idx.indices(len(self))))
            elif isinstance(idx, int):
                new_len = 1
            else:
                t = torch.as_tensor(np.asarray(idx)) if not isinstance(idx, torch.Tensor) else idx
                new_len = int(t.sum()) if t.dtype == torch.bool else int(t.numel())
        out._batch_size = (new_len,) + tuple(self._batch_size[1:])
        return out

    def select(self, *keys: str, strict: bool = True) -> "TensorDict":
        out = TensorDict.__new__(TensorDict)
        out._data = {}
        for k in keys:
            if k in self._data:
                out._data[k] = self._data[k]
            elif strict:
                raise KeyError(k)
        out._batch_size = self._batch_size
        return out

    def exclude(self, *keys: str) -> "TensorDict":
        return self.select(*[k for k in self._data if k not in keys])

    # -- whole-dict transforms ---------------------------------------------------------------------
    def _map(self, fn) -> "TensorDict":
        out = TensorDict.__new__(TensorDict)
        out._data = {k: (v if isinstance(v, NonTensor) else fn(v)) for k, v in self._data.items()}
        out._batch_size = self._batch_size
        return out

    def to(self, *args, **kwargs) -> "TensorDict":
        return self._map(lambda t: t.to(*args, **kwargs))

    def cpu(self):
        return self.to("cpu")

    def cuda(self, device=None):
        return self.to("cuda" if device is None else device)

    def clone(self) -> "TensorDict":
        out = self._map(lambda t: t.clone())
        out._data = {k: (NonTensor(copy.deepcopy(v.data)) if isinstance(v, NonTensor) else v) for k, v in out._data.items()}
        return out

    def contiguous(self) -> "TensorDict":
        return self._map(lambda t: t if isinstance(t, NestedRows) else t.contiguous())

    def consolidate(self) -> "TensorDict":
        return self.contiguous()

    def pin_memory(self) -> "TensorDict":
        def pin(t):
            if isinstance(t, NestedRows):
                return NestedRows(t.values.pin_memory(), t.offsets)
            return t.pin_memory()

        return self._map(pin)

    def chunk(self, chunks: int, dim: int = 0) -> list["TensorDict"]:
        assert dim == 0
        n = len(self)
        size = (n + chunks - 1) // chunks if n else 0
        return [self[i : i + size] for i in range(0, n, size)] if size else [self]

    def split(self, split_size: int, dim: int = 0) -> list["TensorDict"]:
        assert dim == 0
        return [self[i : i + split_size] for i in range(0, len(self), split_size)]

    def to_dict(self) -> dict[str, Any]:
        return {k: (v.data if isinstance(v, NonTensor) else v) for k, v in self._data.items()}

    def __repr__(self) -> str:  # pragma: no cover
        inner = ", ".join(
            f"{k}: {tuple(v.shape) if isinstance(v, torch.Tensor) else v!r}" for k, v in self._data.items()
        )
        return f"TensorDict(batch_size={self._batch_size}, {{{inner}}})"

    # -- pickling: move to CPU-contiguous storage so the object store never holds CUDA handles -------
    def __getstate__(self):
        return {"batch_size": self._batch_size, "data": self._data}

    def __setstate__(self, state):
        self._batch_size = tuple(state["batch_size"])
        self._data = state["data"]


# ------------------------------------------------------------------------------------------------
# free functions
# ------------------------------------------------------------------------------------------------
def cat_tensordicts(tds: Sequence[TensorDict]) -> TensorDict:
    if len(tds) == 0:
        return TensorDict({}, batch_size=(0,))
    keys = tds[0].keys()
    out = TensorDict.__new__(TensorDict)
    out._data = {}
    for k in keys:
        vals = [td._data[k] for td in tds]
        if isinstance(vals[0], NonTensor):
            out._data[k] = vals[0]
        elif isinstance(vals[0], NestedRows):
            rows: list[torch.Tensor] = []
            for v in vals:
                rows.extend(v.unbind())
            out._data[k] = NestedRows.from_list(rows)
        else:
            out._data[k] = torch.cat(vals, dim=0)
    out._batch_size = (sum(len(td) for td in tds),) + tuple(tds[0]._batch_size[1:])
    return out


concat_tensordict = cat_tensordicts


def chunk_tensordict(td: TensorDict, chunks: int) -> list[TensorDict]:
    assert len(td) % chunks == 0, f"batch {len(td)} not divisible into {chunks} chunks"
    size = len(td) // chunks
    return [td[i * size : (i + 1) * size] for i in range(chunks)]


def index_select_tensor_dict(td: TensorDict, idx) -> TensorDict:
    return td[idx]


def get_tensordict(tensor_dict: Mapping[str, Any], non_tensor_dict: Mapping[str, Any] | None = None) -> TensorDict:
    """Build a TensorDict; python lists of tensors become jagged entries, other values non-tensors."""
    src: dict[str, Any] = {}
    bsz = None
    for k, v in tensor_dict.items():
        if isinstance(v, (list, tuple)) and len(v) and all(isinstance(x, torch.Tensor) for x in v):
            v = NestedRows.from_list(list(v))
        if isinstance(v, (torch.Tensor, NestedRows)):
            n = _batch_len(v)
            if bsz is None:
                bsz = n
            assert n == bsz, f"batch mismatch on '{k}': {n} vs {bsz}"
            src[k] = v
        else:
            src[k] = NonTensor(v)
    for k, v in (non_tensor_dict or {}).items():
        src[k] = NonTensor(v)
    return TensorDict(src, batch_size=(bsz or 0,))


def assign_non_tensor(td: TensorDict, **kwargs) -> TensorDict:
    for k, v in kwargs.items():
        td[k] = NonTensor(v)
    return td


def get_non_tensor_data(td: TensorDict, key: str, default=None):
    return td.get(key, default)


def make_iterator(td: TensorDict, mini_batch_size: int, epochs: int = 1, seed: int | None = None,
                  shuffle: bool = False, drop_last: bool = True) -> Iterator[TensorDict]:
    """Yield mini-batches of ``mini_batch_size`` rows for ``epochs`` passes (seeded shuffle per epoch)."""
    n = len(td)
    assert n % mini_batch_size == 0 or not drop_last, f"{n} % {mini_batch_size} != 0"
    gen = torch.Generator()
    if seed is not None:
        gen.manual_seed(int(seed))
    for _ in range(epochs):
        order = torch.randperm(n, generator=gen) if shuffle else torch.arange(n)
        for s in range(0, n - (n % mini_batch_size if drop_last else 0), mini_batch_size):
            idx = order[s : s + mini_batch_size]
            yield td[idx] if shuffle else td[s : s + mini_batch_size]


def pad_to_divisor(td: TensorDict, divisor: int) -> tuple[TensorDict, int]:
    n = len(td)
    pad = (-n) % divisor
    if pad == 0 or n == 0:
        return td, 0
    reps = [td]
    left = pad
    while left > 0:
        take = min(left, n)
        reps.append(td[:take])
        left -= take
    return cat_tensordicts(reps), pad


def unpad(td: TensorDict, pad: int) -> TensorDict:
    return td[: len(td) - pad] if pad else td
