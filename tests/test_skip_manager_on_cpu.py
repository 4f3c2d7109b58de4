"""Rollout skip: the second run replays dumped generations instead of calling the generator."""
import torch

from verl_b200.protocol import DataProto
from verl_b200.utils.skip import SkipManager


class Gen:
    calls = 0

    @SkipManager.annotate("rollout")
    def generate_sequences(self, prompts):
        Gen.calls += 1
        return DataProto.from_dict(tensors={"responses": prompts.batch["input_ids"] + Gen.calls})


def test_rollout_skip_dump_and_replay(tmp_path):
    p = DataProto.from_dict(tensors={"input_ids": torch.arange(6).view(2, 3)})
    SkipManager.reset()
    assert Gen().generate_sequences(p).batch["responses"][0, 0] == 1  # inert before init
    cfg = {"trainer": {"project_name": "p", "experiment_name": "e"}, "skip": {"rollout": {"enable": True, "dump_dir": str(tmp_path)}}}
    SkipManager.init(cfg)
    SkipManager.set_step(1)
    first = Gen().generate_sequences(p)
    assert Gen.calls == 2 and (tmp_path / "p" / "e" / "step_1" / "gen_batch.pkl").exists()
    again = Gen().generate_sequences(p)
    assert Gen.calls == 2 and torch.equal(again.batch["responses"], first.batch["responses"])
    SkipManager.set_step(2)
    Gen().generate_sequences(p)
    assert Gen.calls == 3
    cfg["skip"]["rollout"]["action_on_miss"] = "latest"
    SkipManager.init(cfg)
    SkipManager.set_step(7)
    assert torch.equal(Gen().generate_sequences(p).batch["responses"], p.batch["input_ids"] + 3) and Gen.calls == 3
    SkipManager.reset()
