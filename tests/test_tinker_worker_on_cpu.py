"""Tinker-style primitives: gradient accumulation over two forward_backward calls, client-chosen lr per step."""
import pytest
import torch


def test_tinker_training_worker_accumulates_and_steps(monkeypatch):
    monkeypatch.setenv("VERL_ENGINE_DEVICE", "cpu")
    from functools import partial

    from verl_b200.models import get_preset
    from verl_b200.protocol import DataProto
    from verl_b200.workers.config import FSDPEngineConfig, HFModelConfig, OptimizerConfig, TrainingWorkerConfig
    from verl_b200.workers.engine_workers_tinker import TinkerTrainingWorker, apply_optim_step_params
    from verl_b200.workers.utils.losses import sft_loss

    mc = HFModelConfig(path="tiny-qwen2", load_weights=False)
    w = TinkerTrainingWorker(TrainingWorkerConfig(model_type="language_model", model_config=mc, engine_config=FSDPEngineConfig(seed=1),
                                                  optimizer_config=OptimizerConfig(lr=1e-3)))
    w.reset()
    w.set_loss_fn(partial(sft_loss, None))
    ids = torch.randint(3, 500, (4, 24), generator=torch.Generator().manual_seed(0))
    am = torch.ones_like(ids)
    batch = DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": am, "responses": ids[:, 8:], "response_mask": am[:, 8:]})
    before = w.engine.params.flat.clone()
    w.optimizer_zero_grad()
    m1 = w.forward_backward(batch).meta_info["metrics"]
    g1 = w.engine.params.main_grad.clone()
    w.forward_backward(batch)
    assert torch.allclose(w.engine.params.main_grad, 2 * g1, rtol=1e-4, atol=1e-6)  # accumulated, not overwritten
    out = w.optimizer_step({"lr": 0.0})
    assert torch.equal(w.engine.params.flat, before) and out["grad_norm"] > 0  # lr 0: nothing moves
    w.optimizer_zero_grad()
    w.forward_backward(batch)
    w.optimizer_step({"lr": 1e-2, "betas": (0.8, 0.9)})
    assert not torch.equal(w.engine.params.flat, before) and w.engine.optimizer_config.lr == 1e-3  # config restored
    w.optimizer_zero_grad()
    m2 = w.forward_backward(batch).meta_info["metrics"]
    assert m2["loss"] < m1["loss"]
    with pytest.raises(ValueError):
        apply_optim_step_params(w.engine, {"momentum": 0.9})
    with pytest.raises(TypeError):
        apply_optim_step_params(w.engine, {"lr": "fast"})
