"""Statistics over the whole batch (whitening, batch-size scaling, the adaptive KL controller) do not depend on how many
controller-replicated ranks the batch is split over: two gloo ranks against one process on the concatenated batch."""
import os
import socket

import numpy as np
import pytest
import torch

ESTIMATORS = ["gae", "reinforce_plus_plus", "reinforce_plus_plus_baseline", "gpg", "gdpo"]


def _full_batch():
    from verl_b200.protocol import DataProto

    g = torch.Generator().manual_seed(5)
    B, R = 12, 7
    lens = torch.randint(1, R + 1, (B,), generator=g)
    mask = (torch.arange(R).unsqueeze(0) < lens.unsqueeze(1)).float()
    scores = torch.zeros(B, R)
    scores[torch.arange(B), lens - 1] = torch.randint(0, 3, (B,), generator=g).float()
    t = {"response_mask": mask, "token_level_scores": scores, "token_level_rewards": scores.clone(),
         "values": torch.randn(B, R, generator=g) * mask, "old_log_probs": -torch.rand(B, R, generator=g),
         "ref_log_prob": -torch.rand(B, R, generator=g)}
    uid = np.array([f"p{i // 3}" for i in range(B)], dtype=object)
    return DataProto.from_dict(tensors=t, non_tensors={"uid": uid})


def _run(batch, dp):
    from verl_b200.trainer.ppo import core_algos
    from verl_b200.trainer.ppo.ray_trainer import apply_kl_penalty, compute_advantage

    out = {}
    for name in ESTIMATORS:
        b = compute_advantage(batch, name, gamma=0.97, lam=0.9, config={}, dp=dp)
        out[name] = (b.batch["advantages"].clone(), b.batch["returns"].clone())
    ctrl = core_algos.AdaptiveKLController(init_kl_coef=0.2, target_kl=0.1, horizon=50)
    for _ in range(2):
        batch, m = apply_kl_penalty(batch, ctrl, "kl", dp=dp)
    out["kl"] = (ctrl.value, m["actor/reward_kl_penalty"])
    return out


def _proc(rank, world, port, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        import torch.distributed as dist

        from verl_b200.trainer.ppo.ray_trainer import DataParallelView

        dist.init_process_group("gloo", rank=rank, world_size=world)
        full = _full_batch()
        # uneven split on purpose: 9 + 3 rows, whole prompt groups per rank
        lo, hi = (0, 9) if rank == 0 else (9, 12)
        q.put((rank, _run(full[lo:hi], DataParallelView(None, 1))))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_batch_wide_statistics_do_not_depend_on_the_data_parallel_size():
    import torch.multiprocessing as mp

    want = _run(_full_batch(), None)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r, (lo, hi) in enumerate([(0, 9), (9, 12)]):
        assert "error" not in res[r], res[r]["error"]
        for name in ESTIMATORS:
            for got, ref in zip(res[r][name], want[name]):
                assert torch.allclose(got, ref[lo:hi], atol=1e-5), (name, r)
        assert res[r]["kl"][0] == pytest.approx(want["kl"][0], rel=1e-6) and res[r]["kl"][1] == pytest.approx(want["kl"][1], rel=1e-5)
    # and the local statistics would have been different (the test is not vacuous)
    local = _run(_full_batch()[0:9], None)
    assert not torch.allclose(local["gae"][0], want["gae"][0][0:9], atol=1e-4)
