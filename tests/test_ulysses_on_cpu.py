"""Ulysses sequence parallelism on gloo: two ranks sharing each micro-batch reproduce the single-rank update."""
import os
import socket

import torch

from tests.test_model_parallel_engine_on_cpu import _data, _reference


def _proc(rank, world, port, sp, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                          VERL_ENGINE_DEVICE="cpu")
        from functools import partial

        from verl_b200.models import get_preset
        from verl_b200.utils.distributed import initialize_global_process_group
        from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
        from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead
        from verl_b200.workers.utils.losses import sft_loss

        initialize_global_process_group()
        ec = FSDPEngineConfig(seed=7, micro_batch_size_per_gpu=2, ulysses_sequence_parallel_size=sp)
        eng = NativeEngineWithLMHead(get_preset("tiny-llama"), ec, OptimizerConfig(lr=1e-2, clip_grad=0.05))
        eng.initialize()
        dp = world // sp
        data = _data()
        shard = {k: v.chunk(dp)[rank // sp] for k, v in data.items()}
        out = eng.train_batch(dict(shard), partial(sft_loss, None))
        lp = eng.infer_batch(dict(shard))["model_output"]["log_probs"]
        q.put((rank, {"grad_norm": float(out["metrics"]["grad_norm"]), "flat": eng.params.flat.float().numpy(), "lp": lp.float().numpy()}))
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_sequence_parallel_matches_single_rank():
    import torch.multiprocessing as mp

    ref_norm, ref_lp, ref_flat = _reference()
    for world, sp in ((2, 2), (4, 2)):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        ps = [ctx.Process(target=_proc, args=(r, world, port, sp, q)) for r in range(world)]
        for p in ps:
            p.start()
        res = dict(q.get(timeout=300) for _ in range(world))
        for p in ps:
            p.join(timeout=30)
        rows = ref_lp.chunk(world // sp)
        for r in range(world):
            assert "error" not in res[r], res[r]["error"]
            assert abs(res[r]["grad_norm"] - ref_norm) < 2e-4 * max(1.0, ref_norm), (world, r, res[r]["grad_norm"], ref_norm)
            n = ref_flat.numel()  # the multi-rank buffer is padded to a multiple of the world size
            assert torch.allclose(torch.from_numpy(res[r]["flat"])[:n], ref_flat.float(), atol=3e-4)
            assert torch.allclose(torch.from_numpy(res[r]["lp"]), rows[r // sp], atol=1e-4)
