"""A merged model directory is accepted only when it is a complete Hugging Face model."""
import json
import os

import pytest
import torch
from safetensors.torch import save_file

from verl_b200.model_merger.output_validation import read_safetensors_names, validate_hf_model_output


def _write_cfg(d):
    (d / "config.json").write_text(json.dumps({"model_type": "qwen2"}))


def test_single_file_and_sharded_outputs_pass(tmp_path):
    a = tmp_path / "single"
    a.mkdir()
    _write_cfg(a)
    save_file({"w": torch.ones(2, 2), "b": torch.zeros(2)}, str(a / "model.safetensors"))
    assert read_safetensors_names(a / "model.safetensors") == {"w", "b"}
    validate_hf_model_output(a)
    b = tmp_path / "sharded"
    b.mkdir()
    _write_cfg(b)
    save_file({"w": torch.ones(2, 2)}, str(b / "model-00001-of-00002.safetensors"))
    save_file({"b": torch.zeros(2)}, str(b / "model-00002-of-00002.safetensors"))
    (b / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"w": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}))
    validate_hf_model_output(str(b))


def test_every_kind_of_incomplete_output_is_named(tmp_path):
    d = tmp_path / "out"
    d.mkdir()
    with pytest.raises(RuntimeError, match=r"missing or empty config.json.*no complete model weights"):
        validate_hf_model_output(d)
    (d / "config.json").write_text("[1, 2]")
    with pytest.raises(RuntimeError, match="must contain a JSON object"):
        validate_hf_model_output(d)
    _write_cfg(d)
    # an index that points outside the directory, at a missing shard, at an empty shard
    for wm, msg in (({"w": "../evil.safetensors"}, "unsafe shard paths"), ({"w": "/abs.safetensors"}, "unsafe shard paths"),
                    ({"w": "gone.safetensors"}, "missing or empty shards"), ({}, "no non-empty weight_map"), ({"w": 3}, "invalid shard names")):
        (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
        with pytest.raises(RuntimeError, match=msg):
            validate_hf_model_output(d)
    (d / "empty.safetensors").write_bytes(b"")
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"w": "empty.safetensors"}}))
    with pytest.raises(RuntimeError, match="missing or empty shards"):
        validate_hf_model_output(d)
    # a shard that exists but does not hold what the index says, and one whose header is cut off
    save_file({"other": torch.ones(1)}, str(d / "s1.safetensors"))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"w": "s1.safetensors"}}))
    with pytest.raises(RuntimeError, match="lacks 1 tensors"):
        validate_hf_model_output(d)
    whole = (d / "s1.safetensors").read_bytes()
    (d / "s2.safetensors").write_bytes(whole[:12])
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"other": "s2.safetensors"}}))
    with pytest.raises(RuntimeError, match="truncated header"):
        validate_hf_model_output(d)
    (d / "model.safetensors.index.json").write_text("{not json")
    with pytest.raises(RuntimeError, match="invalid model.safetensors.index.json"):
        validate_hf_model_output(d)
    # a broken index does not matter once a complete single-file model is there
    save_file({"w": torch.ones(1)}, str(d / "model.safetensors"))
    validate_hf_model_output(d)
