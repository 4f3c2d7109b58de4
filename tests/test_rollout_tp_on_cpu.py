"""Tensor-parallel rollout over in-place weight shards: two gloo ranks generate exactly what one full engine does."""
import os
import socket

import torch


def _proc(rank, port, q):
    try:
        import torch.distributed as dist

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=2)
        from verl_b200.models import FlatParams, get_preset
        from verl_b200.workers.rollout.native.engine import RolloutEngine, SamplingParams

        cfg = get_preset("tiny-qwen2")
        P = FlatParams(cfg, dtype=torch.float32)
        P.init_weights(seed=3, std=0.1)
        prompts = [[5, 6, 7, 8, 9], [10, 11, 12], [20, 21, 22, 23, 24, 25, 26], [3, 4]]
        sp = SamplingParams(temperature=1.0, max_tokens=7, seed=11)
        tp = RolloutEngine(cfg, P, max_num_seqs=3, max_model_len=64, block_size=8, eos_token_id=-1, tp_group=dist.group.WORLD)
        outs = tp.generate(prompts, sp)
        assert tp.kv.shape[4] == cfg.num_key_value_heads // 2
        full = RolloutEngine(cfg, P, max_num_seqs=3, max_model_len=64, block_size=8, eos_token_id=-1)
        ref = full.generate(prompts, sp)
        ok = all(a.token_ids == b.token_ids for a, b in zip(outs, ref))
        lp = max(abs(x - y) for a, b in zip(outs, ref) for x, y in zip(a.log_probs, b.log_probs))
        q.put((rank, ok, lp, [o.token_ids for o in outs]))
        dist.destroy_process_group()
    except Exception:
        import traceback

        q.put((rank, False, traceback.format_exc(), None))


def test_tp2_rollout_matches_single_engine():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for rank, ok, lp, toks in res:
        assert ok, lp
        assert lp < 1e-4
    assert res[0][3] == res[1][3]  # both ranks hold identical outputs
