"""Every example script's overrides compose against the configuration tree it targets (no training is run)."""
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = sorted(glob.glob(os.path.join(ROOT, "examples", "*", "*.sh")))


def _overrides(path):
    text = open(path).read()
    entry = re.search(r"-m (verl_b200\.[\w.]+)", text).group(1)
    body = text[text.index(entry) + len(entry):].replace("\\\n", " ")
    toks = re.findall(r"""(?:[^\s"']+|"[^"]*"|'[^']*')+""", body)
    out = []
    for t in toks:
        t = t.strip()
        if "=" not in t or t.startswith(('"${', "${")):
            continue
        k, v = t.split("=", 1)
        v = v.strip("'\"")
        v = re.sub(r"\$\(\(.*?\)\)", "512", v)                 # shell arithmetic
        v = re.sub(r"\$\{?\w+\}?", "8" if re.search(r"size|NGPUS|gpus|step", t) else "tiny-qwen2", v)   # shell variables
        out.append(f"{k}={v}")
    # what the synthetic-data branch of the scripts adds
    if "main_ppo" in entry or "fully_async" in entry:
        out += ["data.synthetic.num_prompts=64", "data.synthetic.prompt_length=16", "reward_model.reward_manager=token_rule"]
    return entry, out


def test_there_are_scripts_for_the_named_configurations():
    names = {os.path.relpath(p, os.path.join(ROOT, "examples")) for p in SCRIPTS}
    assert {"grpo_trainer/run_qwen2_5_7b.sh", "grpo_trainer/run_qwen2_5_0_5b.sh", "grpo_trainer/run_qwen3_30b_a3b_ep8.sh",
            "ppo_trainer/run_llama3_1_8b_tp4_pp2.sh", "sft/run_sft.sh", "distillation/run_on_policy_distillation.sh",
            "fully_async/run_fully_async.sh"} <= names
    for p in SCRIPTS:
        assert os.access(p, os.X_OK) and open(p).readline().startswith("#!/usr/bin/env bash")


@pytest.mark.parametrize("path", SCRIPTS, ids=[os.path.basename(p) for p in SCRIPTS])
def test_overrides_compose(path):
    from verl_b200.trainer.config import CONFIG_DIR
    from verl_b200.utils.config import load_config

    entry, ov = _overrides(path)
    cfg = load_config(CONFIG_DIR, "sft_trainer_engine" if entry.endswith("sft_trainer") else "ppo_trainer", ov)
    for o in ov:
        k = o.split("=", 1)[0].lstrip("+")
        if "@" in k:
            continue
        node = cfg
        for part in k.split("."):
            assert part in node, f"{os.path.basename(path)}: override {o!r} does not land in the configuration tree"
            node = node[part]
    if "tp4_pp2" in path:
        assert cfg.actor_rollout_ref.actor.strategy == "megatron" and cfg.critic.strategy == "megatron"
        assert int(cfg.actor_rollout_ref.actor.megatron.tensor_model_parallel_size) == 4
    if "ep8" in path:
        assert int(cfg.actor_rollout_ref.actor.megatron.expert_model_parallel_size) == 8
    if "distillation" in path:
        assert cfg.distillation.enabled in (True, "true") and cfg.distillation.distillation_loss.loss_mode == "k3"
