#!/usr/bin/env bash
# GRPO on Qwen3-30B-A3B: the experts of every layer are sharded over the 8 data-parallel ranks (expert parallelism); token
# exchange between the ranks goes through peer memory.
set -euo pipefail
NGPUS=${NGPUS:-8}
MODEL=${MODEL:-Qwen/Qwen3-30B-A3B}
TRAIN=${TRAIN:-}
DATA_ARGS=()
if [ -n "$TRAIN" ]; then DATA_ARGS+=("data.train_files=$TRAIN"); else DATA_ARGS+=("data.synthetic.num_prompts=65536" "data.synthetic.prompt_length=1024" "reward_model.reward_manager=token_rule"); fi

python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPUS" --master-addr 127.0.0.1 -m verl_b200.trainer.main_ppo \
    algorithm.adv_estimator=grpo \
    actor@actor_rollout_ref.actor=megatron_actor \
    "${DATA_ARGS[@]}" \
    data.train_batch_size=$((32 * NGPUS)) data.max_prompt_length=1024 data.max_response_length=2048 \
    actor_rollout_ref.model.path="$MODEL" \
    actor_rollout_ref.actor.megatron.tensor_model_parallel_size=1 \
    actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=1 \
    actor_rollout_ref.actor.megatron.expert_model_parallel_size="$NGPUS" \
    actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=$((32 * NGPUS)) \
    actor_rollout_ref.actor.use_dynamic_bsz=true actor_rollout_ref.actor.ppo_max_token_len_per_gpu=16384 \
    actor_rollout_ref.actor.use_kl_loss=true actor_rollout_ref.actor.kl_loss_coef=0.001 \
    actor_rollout_ref.rollout.n=5 actor_rollout_ref.rollout.tensor_model_parallel_size=1 \
    actor_rollout_ref.rollout.gpu_memory_utilization=0.45 \
    trainer.worker_group=spmd trainer.n_gpus_per_node="$NGPUS" trainer.nnodes=1 \
    trainer.total_epochs=15 trainer.save_freq=-1 trainer.test_freq=-1 trainer.logger='[console]' \
    trainer.project_name=verl_b200_examples trainer.experiment_name=qwen3_30b_a3b_grpo_ep8 "$@"
