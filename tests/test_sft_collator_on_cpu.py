"""SFT collation by pad mode: stacked fixed-length samples, jagged variable-length ones."""
import pytest
import torch

from verl_b200.utils.dataset.dataset_utils import DatasetPadMode, SFTTensorCollator, pad_sample


def _sample(n, extra=None):
    s = {"input_ids": torch.arange(1, n + 1), "loss_mask": torch.ones(n, dtype=torch.int64), "position_ids": torch.arange(n), "tag": f"s{n}"}
    s.update(extra or {})
    return s


def test_variable_length_samples_become_jagged_rows():
    out = SFTTensorCollator(DatasetPadMode.NO_PADDING)([_sample(3), _sample(5), _sample(2)])
    ids = out["input_ids"]
    assert ids.is_nested and [int(r.shape[0]) for r in ids.unbind()] == [3, 5, 2]
    assert torch.equal(ids.values(), torch.tensor([1, 2, 3, 1, 2, 3, 4, 5, 1, 2])) and ids.offsets().tolist() == [0, 3, 8, 10]
    assert out["tag"] == ["s3", "s5", "s2"] and out["loss_mask"].values().sum() == 10


def test_fixed_length_samples_are_stacked_and_ragged_ones_refused():
    padded = [pad_sample(_sample(3), 6, pad_token_id=9), pad_sample(_sample(5), 6, pad_token_id=9)]
    out = SFTTensorCollator("right")(padded)
    assert out["input_ids"].shape == (2, 6) and out["input_ids"][0].tolist() == [1, 2, 3, 9, 9, 9]
    assert out["attention_mask"].tolist() == [[1, 1, 1, 0, 0, 0], [1, 1, 1, 1, 1, 0]] and out["loss_mask"][0].tolist() == [1, 1, 1, 0, 0, 0]
    assert out["tag"] == ["s3", "s5"]
    with pytest.raises(ValueError, match="different shapes"):
        SFTTensorCollator(DatasetPadMode.LEFT_RIGHT)([_sample(3), _sample(4)])
    with pytest.raises(ValueError, match="does not fit"):
        pad_sample(_sample(7), 6)
    with pytest.raises(ValueError):
        SFTTensorCollator("diagonal")
