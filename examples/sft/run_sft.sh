#!/usr/bin/env bash
# Multi-turn SFT: parquet / jsonl rows with a `messages` column (and optionally `tools`); the loss covers assistant turns.
set -euo pipefail
NGPUS=${NGPUS:-8}
MODEL=${MODEL:-Qwen/Qwen2.5-7B-Instruct}
TRAIN=${TRAIN:?set TRAIN to a parquet or jsonl file with a messages column}
VAL=${VAL:-}
EXTRA=()
if [ -n "$VAL" ]; then EXTRA+=("data.val_files=$VAL" "trainer.test_freq=100"); fi

python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPUS" --master-addr 127.0.0.1 -m verl_b200.trainer.sft_trainer \
    model.path="$MODEL" \
    data.train_files="$TRAIN" "${EXTRA[@]}" \
    data.train_batch_size=256 data.max_length=4096 data.truncation=right \
    data.use_dynamic_bsz=true data.max_token_len_per_gpu=16384 \
    optim.lr=1e-5 optim.lr_scheduler_type=cosine optim.lr_warmup_steps_ratio=0.05 \
    engine.enable_gradient_checkpointing=true \
    trainer.n_gpus_per_node="$NGPUS" trainer.total_epochs=2 trainer.save_freq=500 \
    trainer.project_name=verl_b200_examples trainer.experiment_name=sft "$@"
