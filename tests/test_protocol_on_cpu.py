"""DataProto semantics (modelled on the reference's tests/test_protocol_on_cpu.py)."""
import pickle

import numpy as np
import pytest
import torch

from verl_b200 import DataProto, pad_dataproto_to_divisor, unpad_dataproto
from verl_b200.protocol import DataProtoFuture, fold_batch_dim, unfold_batch_dim, union_tensor_dict
from verl_b200.utils.tensordict_lite import NestedRows, TensorDict, cat_tensordicts


def make(n=6):
    return DataProto.from_dict(tensors={"obs": torch.arange(n * 3).view(n, 3), "act": torch.arange(n)},
                               non_tensors={"label": np.array([f"s{i}" for i in range(n)], dtype=object)},
                               meta_info={"name": "abc"})


def test_len_getitem_slice():
    d = make()
    assert len(d) == 6
    assert d[2].batch["act"].item() == 2 and d[2].non_tensor_batch["label"] == "s2"
    s = d[1:4]
    assert len(s) == 3 and s.batch["act"].tolist() == [1, 2, 3] and s.non_tensor_batch["label"].tolist() == ["s1", "s2", "s3"]
    idx = d[[0, 5]]
    assert idx.batch["act"].tolist() == [0, 5]
    m = d[torch.tensor([True, False, True, False, False, False])]
    assert m.batch["act"].tolist() == [0, 2]


def test_chunk_concat_roundtrip():
    d = make()
    parts = d.chunk(3)
    assert [len(p) for p in parts] == [2, 2, 2]
    back = DataProto.concat(parts)
    assert torch.equal(back.batch["obs"], d.batch["obs"]) and back.non_tensor_batch["label"].tolist() == d.non_tensor_batch["label"].tolist()
    with pytest.raises(AssertionError):
        d.chunk(4)


def test_concat_merges_metrics():
    a, b = make(2), make(2)
    a.meta_info["metrics"] = {"loss": 1.0}
    b.meta_info["metrics"] = {"loss": 3.0}
    c = DataProto.concat([a, b])
    assert c.meta_info["metrics"] == {"loss": [1.0, 3.0]} and c.meta_info["name"] == "abc"


def test_union_and_conflict():
    d = make()
    e = DataProto.from_dict(tensors={"rew": torch.ones(6)})
    d.union(e)
    assert "rew" in d.batch.keys()
    bad = DataProto.from_dict(tensors={"act": torch.zeros(6, dtype=torch.int64)})
    with pytest.raises(AssertionError):
        d.union(bad)


def test_repeat_interleave_and_not():
    d = make(2)
    r = d.repeat(2, interleave=True)
    assert r.batch["act"].tolist() == [0, 0, 1, 1] and r.non_tensor_batch["label"].tolist() == ["s0", "s0", "s1", "s1"]
    r2 = d.repeat(2, interleave=False)
    assert r2.batch["act"].tolist() == [0, 1, 0, 1]
    r3 = d.sample_level_repeat([1, 3])
    assert r3.batch["act"].tolist() == [0, 1, 1, 1]


def test_pop_select_rename_reorder():
    d = make()
    p = d.pop(batch_keys=["act"], non_tensor_batch_keys=["label"])
    assert "act" not in d.batch.keys() and "label" not in d.non_tensor_batch and len(p) == 6
    d = make()
    s = d.select(batch_keys=["obs"], non_tensor_batch_keys=[])
    assert list(s.batch.keys()) == ["obs"] and s.non_tensor_batch == {}
    d.rename("act", "action")
    assert "action" in d.batch.keys()
    d.reorder(torch.tensor([5, 4, 3, 2, 1, 0]))
    assert d.batch["action"].tolist() == [5, 4, 3, 2, 1, 0] and d.non_tensor_batch["label"][0] == "s5"


def test_padding_helpers():
    d = make(5)
    p, pad = pad_dataproto_to_divisor(d, 4)
    assert len(p) == 8 and pad == 3 and p.batch["act"].tolist() == [0, 1, 2, 3, 4, 0, 1, 2]
    assert len(unpad_dataproto(p, pad)) == 5
    p2, pad2 = pad_dataproto_to_divisor(make(2), 7)  # pad larger than batch: cycles
    assert len(p2) == 7 and pad2 == 5


def test_pickle_and_disk(tmp_path, monkeypatch):
    d = make()
    e = pickle.loads(pickle.dumps(d))
    assert torch.equal(e.batch["obs"], d.batch["obs"]) and e.meta_info == d.meta_info
    monkeypatch.setenv("VERL_DATAPROTO_SERIALIZATION_METHOD", "numpy")
    d2 = DataProto.from_dict(tensors={"x": torch.randn(3, 2).bfloat16(), "y": torch.arange(3)})
    e2 = pickle.loads(pickle.dumps(d2))
    assert e2.batch["x"].dtype == torch.bfloat16 and torch.equal(e2.batch["x"], d2.batch["x"])
    f = tmp_path / "d.pkl"
    d.save_to_disk(str(f))
    assert len(DataProto.load_from_disk(str(f))) == 6


def test_make_iterator_and_split():
    d = make()
    seen = [b.batch["act"].tolist() for b in d.make_iterator(mini_batch_size=2, epochs=2, seed=1)]
    assert len(seen) == 6 and sorted(sum(seen[:3], [])) == list(range(6))
    assert [len(x) for x in d.split(4)] == [4, 2]


def test_fold_unfold_and_column_chunks():
    d = make()
    f = fold_batch_dim(d, 2)
    assert f.batch["obs"].shape == (2, 3, 3)
    u = unfold_batch_dim(f, 2)
    assert torch.equal(u.batch["obs"], d.batch["obs"])
    x = DataProto.from_dict(tensors={"a": torch.arange(8).view(2, 4), "b": torch.tensor([7, 9])})
    y = x.unfold_column_chunks(2, split_keys=["a"])
    assert y.batch["a"].tolist() == [[0, 1], [2, 3], [4, 5], [6, 7]] and y.batch["b"].tolist() == [7, 7, 9, 9]


def test_future_and_tensordict_roundtrip():
    parts = make().chunk(2)
    fut = DataProtoFuture.concat(parts)
    assert len(fut.get()) == 6
    assert [len(c.get()) for c in fut.chunk(3)] == [2, 2, 2]
    td = make().to_tensordict()
    back = DataProto.from_tensordict(td)
    assert back.meta_info["name"] == "abc" and back.non_tensor_batch["label"].tolist()[0] == "s0"


def test_nested_rows():
    rows = [torch.arange(3), torch.arange(5), torch.arange(1)]
    n = NestedRows.from_list(rows)
    assert n.lengths().tolist() == [3, 5, 1] and n.to_padded(pad_value=-1).shape == (3, 5)
    assert n.to_padded(pad_value=-1, left=True)[0].tolist() == [-1, -1, 0, 1, 2]
    td = TensorDict({"x": n, "y": torch.arange(3)})
    c = cat_tensordicts([td[:1], td[1:]])
    assert c["x"].lengths().tolist() == [3, 5, 1]
    padded = torch.arange(12).view(3, 4)
    mask = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 1], [0, 0, 0, 1]])
    assert NestedRows.from_padded(padded, mask).values.tolist() == [0, 1, 4, 5, 6, 7, 11]
