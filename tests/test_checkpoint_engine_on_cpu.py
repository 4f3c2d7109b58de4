"""Weight-sync back-ends: bucket packing round trip, sparse deltas, and a two-process gloo broadcast."""
import asyncio
import os
import socket

import pytest
import torch

from verl_b200.checkpoint_engine import CheckpointEngineRegistry, bucketize, merge_weight_chunks
from verl_b200.checkpoint_engine.delta_checkpoint_engine import apply_delta, encode_delta, tensor_checksum


def _weights():
    g = torch.Generator().manual_seed(0)
    return [("a", torch.randn(7, 5, generator=g)), ("b", torch.randn(300, generator=g).bfloat16()),
            ("c", torch.randint(0, 9, (11,), generator=g)), ("d", torch.randn(2, 3, 4, generator=g))]


@pytest.mark.parametrize("bucket", [64, 200, 1 << 16])
def test_bucket_roundtrip_with_split_tensors(bucket):
    out = dict(merge_weight_chunks(bucketize(_weights(), bucket)))
    for n, t in _weights():
        assert out[n].dtype == t.dtype and out[n].shape == t.shape and torch.equal(out[n], t)


def test_delta_encode_apply_checksum():
    old = torch.randn(1000).bfloat16()
    new = old.clone()
    new[[3, 500, 999]] += 1.0
    idx, val = encode_delta(new, old)
    assert idx.tolist() == [3, 500, 999]
    tgt = old.clone()
    apply_delta(tgt, idx, val)
    assert torch.equal(tgt, new) and tensor_checksum(tgt) == tensor_checksum(new) != tensor_checksum(old)


def test_naive_engine_passes_generator_through():
    eng = CheckpointEngineRegistry.new("naive")

    async def go():
        await eng.send_weights(iter(_weights()))
        return [n async for n, _ in eng.receive_weights()]

    assert asyncio.run(go()) == ["a", "b", "c", "d"]


def _proc(rank, port, backend, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    eng = CheckpointEngineRegistry.new(backend, bucket_size=256, group=None, src=0)
    w = _weights()

    async def run():
        got = {}
        for step in range(2):
            if rank == 0:
                if step == 1:
                    w[0][1][0, 0] += 5.0
                await eng.send_weights(iter(w))
            else:
                async for n, t in eng.receive_weights():
                    got[n] = t.clone()
        return got

    got = asyncio.run(run())
    if rank == 1:
        ref = _weights()
        ref[0][1][0, 0] += 5.0
        q.put(all(torch.equal(got[n], t) for n, t in ref))
    else:
        q.put(getattr(eng, "last_stats", {}))
    dist.destroy_process_group()


@pytest.mark.parametrize("backend", ["nccl", "delta_sharded"])
def test_two_process_sync(backend):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_proc, args=(r, port, backend, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in ps:
        p.join(timeout=30)
    assert True in res
    if backend == "delta_sharded":
        stats = next(r for r in res if isinstance(r, dict))
        assert stats["sent_elements"] == 1  # the second sync shipped exactly the one changed element


def _ring_proc(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    eng = CheckpointEngineRegistry.new("nixl", bucket_size=256, group=None, src=0)  # the relay chain under a transport's name
    w = _weights()

    async def run():
        got = {}
        if rank == 0:
            await eng.send_weights(iter(w))
        else:
            async for n, t in eng.receive_weights():
                got[n] = t.clone()
        return got

    got = asyncio.run(run())
    q.put((rank, rank == 0 or all(torch.equal(got[n], t) for n, t in _weights())))
    dist.destroy_process_group()


def test_relay_chain_delivers_to_every_receiver():
    import torch.multiprocessing as mp

    from verl_b200.checkpoint_engine.ring_checkpoint_engine import RingCheckpointEngine

    assert CheckpointEngineRegistry.get("mooncake") is RingCheckpointEngine and CheckpointEngineRegistry.get("kimi") is RingCheckpointEngine
    tr, ro = RingCheckpointEngine.build_topology(2, 3, [])
    assert tr["rank"] == [0, -1] and ro["rank"] == [1, 2, 3] and ro["world_size"] == [4, 4, 4]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_ring_proc, args=(r, 4, port, q)) for r in range(4)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(4))
    for p in ps:
        p.join(timeout=30)
    assert res == {0: True, 1: True, 2: True, 3: True}
