"""SFT through the single controller: the loss goes down on a tiny model; checkpoints save and resume."""


def test_sft_ray_style_trainer_inprocess(tmp_path, monkeypatch):
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from verl_b200.trainer.sft_trainer_ray import main

    args = ['model.path=tiny-qwen2', 'model.load_weights=false', 'data.train_batch_size=8', 'data.max_length=32',
            'data.micro_batch_size_per_gpu=4', 'data.use_dynamic_bsz=false', 'trainer.total_training_steps=6', 'trainer.device=cpu',
            'trainer.logger=[]', 'optim.lr=3e-3', 'trainer.n_gpus_per_node=1', 'trainer.total_epochs=10', 'trainer.save_freq=3',
            f'trainer.default_local_dir={tmp_path}', 'trainer.test_freq=3']
    last = main(args)
    assert last["train/loss"] > 0 and "val/loss" in last
    assert (tmp_path / "global_step_6").exists() and (tmp_path / "latest_checkpointed_iteration.txt").read_text() == "6"
    resumed = main([a for a in args if not a.startswith("trainer.total_training_steps")] + ["trainer.total_training_steps=8"])
    assert resumed["train/loss"] < 7.0
