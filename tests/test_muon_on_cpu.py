"""Muon on the range-sharded optimizer: Newton-Schulz quality, the matrix plan, one engine step against the textbook update,
and equality of the two-rank and one-rank runs."""
import math
import os
import socket
from functools import partial

import pytest
import torch

from verl_b200.workers.engine.native.muon import (MuonPlan, adamw_rms_match_scale_factor, muon_scale_factor, newton_schulz)


@pytest.mark.parametrize("shape", [(64, 64), (32, 96), (96, 32)])
def test_newton_schulz_pushes_singular_values_towards_one(shape):
    g = torch.randn(*shape, generator=torch.Generator().manual_seed(0))
    o = newton_schulz(g, steps=5)
    sv = torch.linalg.svdvals(o)
    # (a square Gaussian matrix has a few singular values next to zero, which five steps cannot lift: judge the bulk)
    assert o.shape == g.shape and 0.6 < float(sv.quantile(0.1)) and float(sv.max()) < 1.3
    # same singular vectors as the input: U^T O V is (nearly) diagonal and positive
    u, _, vh = torch.linalg.svd(g, full_matrices=False)
    d = u.t() @ o @ vh.t()
    assert float((d - torch.diag(torch.diagonal(d))).abs().max()) < 2e-2 and float(torch.diagonal(d).quantile(0.1)) > 0.5
    more = torch.linalg.svdvals(newton_schulz(g, steps=30, coefficient_type="simple"))
    assert float((more - 1).abs().quantile(0.9)) < 0.05  # the convergent polynomial lands on one


def test_scale_factors():
    assert muon_scale_factor(64, 256, "spectral") == 16.0 and muon_scale_factor(256, 64, "shape_scaling") == 2.0
    assert muon_scale_factor(64, 256, "shape_scaling") == 1.0 and muon_scale_factor(256, 64, "unit_rms_norm") == 2.0
    assert abs(adamw_rms_match_scale_factor(0.9) - 0.2294) < 1e-4
    with pytest.raises(ValueError):
        muon_scale_factor(2, 2, "bogus")
    # spectral scaling gives a unit-RMS update
    o = newton_schulz(torch.randn(48, 160, generator=torch.Generator().manual_seed(1)), steps=8, coefficient_type="simple")
    rms = float((o * muon_scale_factor(48, 160, "spectral")).pow(2).mean().sqrt())
    assert 0.9 < rms < 1.1


def test_plan_splits_fused_projections_and_balances_work():
    from verl_b200.models import get_preset
    from verl_b200.models.weights import FlatParams

    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32, pad_to=2)
    plan = MuonPlan(P, world=2)
    assert len(plan.matrices) == cfg.num_hidden_layers * 7      # q, k, v, o, gate, up, down
    shapes = sorted({(m.rows, m.cols) for m in plan.matrices})
    assert (cfg.q_size, cfg.hidden_size) in shapes and (cfg.kv_size, cfg.hidden_size) in shapes
    assert (cfg.intermediate_size, cfg.hidden_size) in shapes and (cfg.hidden_size, cfg.intermediate_size) in shapes
    work = [sum(m.cost for m in plan.matrices if m.owner == r) for r in range(2)]
    assert abs(work[0] - work[1]) / max(work) < 0.15
    mask = plan.mask(0, P.numel, "cpu")
    assert int(mask.sum()) == sum(m.numel for m in plan.matrices)
    o = P.offsets["embed_tokens.weight"]
    assert not mask[o : o + 10].any() and not mask[P.offsets["layers.0.input_layernorm.weight"]]
    assert not mask[P.offsets["layers.0.self_attn.qkv_proj.bias"]] and mask[P.offsets["layers.1.mlp.down_proj.weight"]]
    whole = MuonPlan(P, world=1, split_qkv=False, split_gate_up=False)
    assert len(whole.matrices) == cfg.num_hidden_layers * 4


def _data(b=6, L=20, R=12, V=500, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, V, (b, L), generator=g)
    am = torch.ones_like(ids)
    am[1, :3] = 0
    return {"input_ids": ids, "attention_mask": am, "responses": ids[:, -R:], "response_mask": am[:, -R:]}


def _engine(**opt):
    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.models import get_preset
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    kw = dict(lr=2e-2, clip_grad=0.0, optimizer="muon", weight_decay=0.1)
    kw.update(opt)
    eng = NativeEngineWithLMHead(get_preset("tiny-qwen2"), FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=3), OptimizerConfig(**kw))
    eng.initialize()
    return eng


@pytest.mark.parametrize("nesterov", [False, True])
def test_one_engine_step_equals_the_textbook_update(nesterov):
    from verl_b200.workers.utils.losses import sft_loss

    eng = _engine(muon_nesterov=nesterov, muon_match_adamw_update_rms=True)
    oc = eng.optimizer_config
    w0 = {k: v.clone() for k, v in eng.params.views.items()}
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(dict(_data()), partial(sft_loss, None))
    grads = {k: v.main_grad.clone() for k, v in eng.params.views.items()}
    eng.optimizer_step()
    cfg, lr, wd = eng.arch, 2e-2, 0.1
    extra = math.sqrt(0.1 / 1.9)
    worst = 0.0
    for name, w in w0.items():
        g = grads[name]
        layer_matrix = name.startswith("layers.") and w.dim() == 2
        if layer_matrix:
            if name.endswith("qkv_proj.weight"):
                blocks = [(0, cfg.q_size), (cfg.q_size, cfg.kv_size), (cfg.q_size + cfg.kv_size, cfg.kv_size)]
            elif name.endswith("gate_up_proj.weight"):
                blocks = [(0, w.shape[0] // 2), (w.shape[0] // 2, w.shape[0] // 2)]
            else:
                blocks = [(0, w.shape[0])]
            exp = w.clone()
            for r0, nr in blocks:
                gb = g[r0 : r0 + nr]
                u = gb + oc.muon_momentum * gb if nesterov else gb          # momentum starts from zero: m = g
                o = newton_schulz(u, 5) * math.sqrt(max(nr, w.shape[1]))
                exp[r0 : r0 + nr] = w[r0 : r0 + nr] * (1 - lr * wd) - lr * extra * o
        else:                                                              # first AdamW step: m/(1-b1) = g, sqrt(v/(1-b2)) = |g|
            exp = w * (1 - lr * wd) - lr * g / (g.abs() + oc.eps)
        worst = max(worst, float((eng.params.views[name] - exp).abs().max()))
    assert worst < 2e-5, worst


def test_muon_training_reduces_the_loss():
    from verl_b200.workers.utils.losses import sft_loss

    eng = _engine(lr=5e-3, clip_grad=1.0, muon_match_adamw_update_rms=True)
    losses = [float(eng.train_batch(dict(_data()), partial(sft_loss, None))["loss"]) for _ in range(6)]
    assert losses[-1] < 0.8 * losses[0], losses


def _proc(rank, world, port, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        eng = _engine(clip_grad=0.5)
        norms = []
        for step in range(2):
            shard = {k: v.chunk(world)[rank] for k, v in _data(seed=step).items()}
            norms.append(float(eng.train_batch(dict(shard), partial(sft_loss, None))["metrics"]["grad_norm"]))
        q.put((rank, {"flat": eng.params.flat.numpy(), "norms": norms, "state": eng.exp_avg.numel(),
                      "mine": sum(1 for m in eng.muon.matrices if m.owner == rank)}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_two_ranks_equal_one_rank():
    import torch.multiprocessing as mp

    from verl_b200.workers.utils.losses import sft_loss

    ref = _engine(clip_grad=0.5)
    ref_norms = [float(ref.train_batch(dict(_data(seed=s)), partial(sft_loss, None))["metrics"]["grad_norm"]) for s in range(2)]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    n = ref.params.numel
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert 0 <= res[r]["state"] * 2 - n < 1024 and res[r]["mine"] == 7          # half of the state, half of the matrices
        assert all(abs(a - b) < 2e-4 * max(1.0, b) for a, b in zip(res[r]["norms"], ref_norms))
        assert torch.allclose(torch.from_numpy(res[r]["flat"])[:n], ref.params.flat, atol=3e-5), \
            (torch.from_numpy(res[r]["flat"])[:n] - ref.params.flat).abs().max()


def _tp_proc(rank, world, port, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from verl_b200.models import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import McoreEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.base import EngineRegistry
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        eng = EngineRegistry.new("language_model", "megatron", model_config=get_preset("tiny-qwen2"),
                                 engine_config=McoreEngineConfig(seed=7, micro_batch_size_per_gpu=3, tensor_model_parallel_size=2),
                                 optimizer_config=OptimizerConfig(lr=5e-3, optimizer="muon", muon_match_adamw_update_rms=True))
        eng.initialize()
        losses = [float(eng.train_batch(dict(_data()), partial(sft_loss, None))["loss"]) for _ in range(4)]
        shapes = sorted({(m.rows, m.cols) for m in eng.muon.matrices})
        q.put((rank, {"losses": losses, "shapes": shapes}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_tensor_parallel_shards_are_orthogonalised_blockwise():
    import torch.multiprocessing as mp

    from verl_b200.models import get_preset

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_tp_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    cfg = get_preset("tiny-qwen2")
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert res[r]["losses"][-1] < 0.8 * res[r]["losses"][0] and res[r]["losses"] == res[0]["losses"]
        assert (cfg.q_size // 2, cfg.hidden_size) in res[r]["shapes"] and (cfg.hidden_size, cfg.intermediate_size // 2) in res[r]["shapes"]
