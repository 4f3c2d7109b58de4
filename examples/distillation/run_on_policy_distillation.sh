#!/usr/bin/env bash
# On-policy distillation: the student samples, a frozen teacher scores the sampled tokens, the actor trains on the task loss
# plus a reverse-KL estimator (k3) of student against teacher. DISTILL_ONLY=1 drops the task loss.
set -euo pipefail
NGPUS=${NGPUS:-8}
STUDENT=${STUDENT:-Qwen/Qwen2.5-0.5B-Instruct}
TEACHER=${TEACHER:-Qwen/Qwen2.5-7B-Instruct}
TRAIN=${TRAIN:-}
DATA_ARGS=()
if [ -n "$TRAIN" ]; then DATA_ARGS+=("data.train_files=$TRAIN"); else DATA_ARGS+=("data.synthetic.num_prompts=65536" "data.synthetic.prompt_length=512" "reward_model.reward_manager=token_rule"); fi
if [ "${DISTILL_ONLY:-0}" = "1" ]; then DATA_ARGS+=("distillation.distillation_loss.use_task_rewards=false"); fi

python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPUS" --master-addr 127.0.0.1 -m verl_b200.trainer.main_ppo \
    algorithm.adv_estimator=grpo \
    "${DATA_ARGS[@]}" \
    data.train_batch_size=256 data.max_prompt_length=512 data.max_response_length=1024 \
    actor_rollout_ref.model.path="$STUDENT" \
    actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=256 \
    actor_rollout_ref.actor.use_dynamic_bsz=true actor_rollout_ref.actor.ppo_max_token_len_per_gpu=16384 \
    actor_rollout_ref.actor.use_kl_loss=false \
    actor_rollout_ref.rollout.n=4 actor_rollout_ref.rollout.tensor_model_parallel_size=1 \
    distillation.enabled=true distillation.teacher_models.teacher_model.model_path="$TEACHER" \
    distillation.distillation_loss.loss_mode=k3 distillation.distillation_loss.distillation_loss_coef=1.0 \
    trainer.worker_group=spmd trainer.n_gpus_per_node="$NGPUS" trainer.nnodes=1 \
    trainer.total_epochs=15 trainer.save_freq=-1 trainer.test_freq=-1 trainer.logger='[console]' \
    trainer.project_name=verl_b200_examples trainer.experiment_name=on_policy_distillation "$@"
