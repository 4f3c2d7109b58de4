"""Offline evaluation and batch generation entry points on tiny inputs."""
import json

import torch


def test_main_eval_scores_jsonl(tmp_path):
    from verl_b200.trainer.main_eval import main

    rows = [{"data_source": "openai/gsm8k", "responses": ["so #### 4", "#### 5"], "reward_model": {"ground_truth": "4"}},
            {"data_source": "openai/gsm8k", "responses": ["#### 7"], "reward_model": {"ground_truth": "7"}},
            {"data_source": "nq", "responses": ["<answer>x</answer>"], "reward_model": {"ground_truth": {"target": ["y"]}}}]
    p = tmp_path / "gen.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    m = main([f"data.path={p}", "num_workers=1"])
    assert m == {"test_score/openai/gsm8k": 0.75, "test_score/nq": 0.0}


def test_generation_server_spreads_prompts_over_replicas():
    from verl_b200.models import FlatParams, get_preset
    from verl_b200.trainer.main_generation_server import CONFIG_DIR, run_generation
    from verl_b200.utils.config import load_config
    from verl_b200.workers.rollout.native.engine import RolloutEngine

    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    engines = [RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=64, block_size=8, eos_token_id=-1) for _ in range(2)]
    conf = load_config(CONFIG_DIR, "generation", ["data.n_samples=2", "actor_rollout_ref.rollout.temperature=0.0",
                                                  "actor_rollout_ref.rollout.response_length=5", "actor_rollout_ref.rollout.prompt_length=16"])
    prompts = [[5, 6, 7], [8, 9], [10, 11, 12, 13]]
    outs = run_generation(conf, engines=engines, prompts_ids=prompts)
    assert len(outs) == 3 and all(len(g) == 2 and len(g[0]) == 5 for g in outs)
    assert all(g[0] == g[1] for g in outs)  # greedy: both samples agree
    solo = run_generation(conf, engines=engines[:1], prompts_ids=prompts)
    assert solo == outs
