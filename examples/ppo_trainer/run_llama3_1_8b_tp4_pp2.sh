#!/usr/bin/env bash
# PPO with a critic and GAE on Llama-3.1-8B: tensor-parallel 4 x pipeline-parallel 2 training (actor and critic), rollout
# tensor-parallel size 4; the trainer's shards are pushed into the rollout replicas over peer memory.
set -euo pipefail
NGPUS=${NGPUS:-8}
MODEL=${MODEL:-meta-llama/Llama-3.1-8B-Instruct}
TRAIN=${TRAIN:-}
DATA_ARGS=()
if [ -n "$TRAIN" ]; then DATA_ARGS+=("data.train_files=$TRAIN"); else DATA_ARGS+=("data.synthetic.num_prompts=65536" "data.synthetic.prompt_length=512" "reward_model.reward_manager=token_rule"); fi

python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPUS" --master-addr 127.0.0.1 -m verl_b200.trainer.main_ppo \
    algorithm.adv_estimator=gae algorithm.gamma=1.0 algorithm.lam=1.0 \
    actor@actor_rollout_ref.actor=megatron_actor critic@critic=megatron_critic \
    "${DATA_ARGS[@]}" \
    data.train_batch_size=512 data.max_prompt_length=512 data.max_response_length=512 \
    actor_rollout_ref.model.path="$MODEL" critic.model.path="$MODEL" \
    actor_rollout_ref.actor.megatron.tensor_model_parallel_size=4 actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2 \
    critic.megatron.tensor_model_parallel_size=4 critic.megatron.pipeline_model_parallel_size=2 \
    actor_rollout_ref.actor.optim.lr=1e-6 critic.optim.lr=1e-5 \
    actor_rollout_ref.actor.ppo_mini_batch_size=512 critic.ppo_mini_batch_size=512 \
    actor_rollout_ref.actor.use_dynamic_bsz=true actor_rollout_ref.actor.ppo_max_token_len_per_gpu=16384 \
    critic.use_dynamic_bsz=true critic.ppo_max_token_len_per_gpu=16384 \
    actor_rollout_ref.actor.use_kl_loss=false actor_rollout_ref.actor.clip_ratio=0.2 \
    actor_rollout_ref.rollout.n=1 actor_rollout_ref.rollout.tensor_model_parallel_size=4 \
    actor_rollout_ref.rollout.gpu_memory_utilization=0.45 \
    trainer.worker_group=spmd trainer.n_gpus_per_node="$NGPUS" trainer.nnodes=1 \
    trainer.total_epochs=15 trainer.save_freq=-1 trainer.test_freq=-1 trainer.logger='[console]' \
    trainer.project_name=verl_b200_examples trainer.experiment_name=llama3_1_8b_ppo_tp4_pp2 "$@"
