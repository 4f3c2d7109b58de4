#!/usr/bin/env bash
# Fully asynchronous training: the rollouter keeps producing while the trainer consumes; weights are handed over every
# TRIGGER optimizer steps and the rollouter may run ahead by STALENESS x that many samples.
set -euo pipefail
MODEL=${MODEL:-Qwen/Qwen2.5-7B-Instruct}
TRAIN=${TRAIN:-}
TRIGGER=${TRIGGER:-4}
STALENESS=${STALENESS:-0.5}
DATA_ARGS=()
if [ -n "$TRAIN" ]; then DATA_ARGS+=("data.train_files=$TRAIN"); else DATA_ARGS+=("data.synthetic.num_prompts=65536" "data.synthetic.prompt_length=1024" "reward_model.reward_manager=token_rule"); fi

python -m verl_b200.experimental.fully_async_policy.fully_async_main \
    algorithm.adv_estimator=grpo \
    "${DATA_ARGS[@]}" \
    data.train_batch_size=64 data.max_prompt_length=1024 data.max_response_length=2048 \
    actor_rollout_ref.model.path="$MODEL" \
    actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=64 \
    actor_rollout_ref.actor.use_dynamic_bsz=true actor_rollout_ref.actor.ppo_max_token_len_per_gpu=16384 \
    actor_rollout_ref.actor.use_kl_loss=true actor_rollout_ref.actor.kl_loss_coef=0.001 \
    actor_rollout_ref.rollout.n=5 actor_rollout_ref.rollout.tensor_model_parallel_size=1 \
    +async_training.require_batches=1 +async_training.trigger_parameter_sync_step="$TRIGGER" \
    +async_training.staleness_threshold="$STALENESS" \
    trainer.n_gpus_per_node=1 trainer.nnodes=1 trainer.worker_group=inprocess \
    trainer.total_training_steps=1000 trainer.save_freq=100 trainer.test_freq=-1 trainer.logger='[console]' \
    trainer.project_name=verl_b200_examples trainer.experiment_name=fully_async "$@"
