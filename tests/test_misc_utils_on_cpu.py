"""Small utilities: paths, time limits, dictionaries, dynamic enums, addresses, precision names, debug metrics."""
import asyncio
import os
import time

import pytest
import torch


def test_fs_and_hdfs_io_on_local_paths(tmp_path):
    from verl_b200.utils import fs, hdfs_io

    src = tmp_path / "src"
    (src / "sub").mkdir(parents=True)
    (src / "a.txt").write_text("hello")
    (src / "sub" / "b.bin").write_bytes(b"\x00" * 100)
    assert not fs.is_non_local(str(src)) and fs.is_non_local("hdfs://nn/path")
    assert fs.copy_to_local(str(src)) == str(src)
    dst = tmp_path / "dst"
    assert hdfs_io.copy(str(src), str(dst)) and fs.verify_copy(str(src), str(dst))
    (dst / "a.txt").write_text("hello!")
    assert not fs.verify_copy(str(src), str(dst))
    p1, p2 = fs.get_local_temp_path("hdfs://x/a/model", str(tmp_path)), fs.get_local_temp_path("hdfs://x/b/model", str(tmp_path))
    assert p1 != p2 and os.path.basename(p1) == os.path.basename(p2) == "model"
    shm = fs.copy_to_shm(str(src))
    assert fs.verify_copy(str(src), shm)
    assert hdfs_io.exists(str(src)) and not hdfs_io.exists(str(tmp_path / "nope"))
    assert os.path.isdir(fs.local_mkdir_safe(str(tmp_path / "x" / "y")))


def _slow(t):
    time.sleep(t)
    return t


def test_timeout_limit_process_and_signal():
    from verl_b200.utils.py_functional import timeout_limit

    assert timeout_limit(5.0)(_slow)(0.01) == 0.01
    with pytest.raises(TimeoutError):
        timeout_limit(0.2)(_slow)(5.0)
    with pytest.raises(TimeoutError):
        timeout_limit(0.2, use_signals=True)(_slow)(5.0)

    def boom():
        raise ValueError("x")

    with pytest.raises(ValueError):
        timeout_limit(5.0)(boom)()


from verl_b200.utils.py_functional import DynamicEnum as _DynamicEnum


class _Role(_DynamicEnum):
    _registry, _next_value = {}, 0


def test_dict_helpers_and_dynamic_enum():
    from verl_b200.utils.py_functional import (DynamicEnum, NestedNamespace, append_to_dict, list_of_dict_to_dict_of_list,
                                                rename_dict, temp_env_var, union_two_dict)

    assert union_two_dict({"a": 1}, {"b": 2}) == {"a": 1, "b": 2}
    with pytest.raises(AssertionError):
        union_two_dict({"a": 1}, {"a": 2})
    d = {}
    append_to_dict(d, {"x": 1, "y": [1, 2]}, prefix="m/")
    append_to_dict(d, {"x": 2, "y": [3]}, prefix="m/")
    assert d == {"m/x": [1, 2], "m/y": [1, 2, 3]} and rename_dict({"a": 1}, "p/") == {"p/a": 1}
    ns = NestedNamespace({"a": {"b": [{"c": 3}]}})
    assert ns.a.b[0].c == 3
    assert list_of_dict_to_dict_of_list([{"a": 1}, {"a": 2}]) == {"a": [1, 2]}

    Role = _Role
    actor = Role.register("actor")
    Role.register("critic")
    assert Role.ACTOR is actor and Role["CRITIC"].value == 1 and Role.names() == ["ACTOR", "CRITIC"] and actor in Role
    import pickle

    assert pickle.loads(pickle.dumps(actor)) is actor
    Role.remove("critic")
    assert Role.from_name("critic") is None
    with temp_env_var("VB_TEST_ENV", "1"):
        assert os.environ["VB_TEST_ENV"] == "1"
    assert "VB_TEST_ENV" not in os.environ


def test_net_precision_logger_ray_utils(capsys):
    from verl_b200.utils.logger import LocalLogger, concat_dict_to_str
    from verl_b200.utils.net_utils import get_free_port, is_ipv4, is_ipv6
    from verl_b200.utils.ray_utils import auto_await, ray_noset_visible_devices
    from verl_b200.utils.torch_dtypes import PrecisionType

    assert is_ipv4("10.0.0.1") and not is_ipv4("::1") and is_ipv6("[::1]") and not is_ipv6("host")
    port, sock = get_free_port("127.0.0.1", with_alive_sock=True)
    assert 0 < port < 65536 and sock is not None
    sock.close()
    assert PrecisionType.to_dtype("bf16") is torch.bfloat16 and PrecisionType.is_fp16(16) and PrecisionType.to_str(torch.float32) == "fp32"
    assert concat_dict_to_str({"a": 1.0, "s": "x"}, 3) == "step:3 - a:1.000"
    LocalLogger().log({"loss": 0.5}, 1)
    assert "loss:0.500" in capsys.readouterr().out
    assert ray_noset_visible_devices({"RAY_EXPERIMENTAL_NOSET_CUDA_VISIBLE_DEVICES": "1"}) and not ray_noset_visible_devices({})

    @auto_await
    async def f(x):
        await asyncio.sleep(0)
        return x + 1

    assert f(1) == 2


def test_debug_metrics_and_tracker(tmp_path, monkeypatch):
    from verl_b200.protocol import DataProto
    from verl_b200.utils.debug import calculate_debug_metrics, calculate_token_list_diff, dump_data, get_trajectory_tracker

    lp = torch.log(torch.tensor([[0.5, 0.25, 0.1], [0.3, 0.3, 0.3]]))
    lp2 = lp.clone()
    lp2[0, 0] = torch.log(torch.tensor(0.4))
    mask = torch.tensor([[1, 1, 0], [1, 1, 1]])
    data = DataProto.from_dict({"rollout_log_probs": lp, "old_log_probs": lp2, "response_mask": mask, "responses": torch.zeros(2, 3, dtype=torch.long)})
    m = calculate_debug_metrics(data)
    assert abs(m["training/rollout_probs_diff_max"] - 0.1) < 1e-6 and m["training/rollout_actor_probs_pearson_corr"] > 0.9
    d = calculate_token_list_diff(torch.tensor([[1, 2, 3]]), torch.tensor([[1, 5, 9]]), torch.tensor([[1, 1, 0]]))
    assert abs(d.item() - 0.5) < 1e-6
    monkeypatch.setenv("VERL_ENABLE_TRACKER", "1")
    monkeypatch.setenv("VERL_TRACKER_HDFS_DIR", str(tmp_path / "trk"))
    import verl_b200.utils.debug.trajectory_tracker as tt

    tt._TRACKER = None
    dump_data({"x": torch.ones(3)}, "step0")
    (path,) = get_trajectory_tracker().wait_for_hdfs()
    assert torch.equal(torch.load(path)["x"], torch.ones(3))
    tt._TRACKER = None


def _ulysses_proc(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        import torch.distributed as dist

        from verl_b200.utils import ulysses as U

        dist.init_process_group("gloo", rank=rank, world_size=world)
        U.set_ulysses_sequence_parallel_group(dist.group.WORLD)
        g = torch.Generator().manual_seed(0)
        full = torch.randn(1, 6, 4, 8, generator=g)  # [b, seq, heads, dim]
        local = U.slice_input_tensor(full, dim=1).clone().requires_grad_(True)
        x = U.gather_seq_scatter_heads(local, seq_dim=1, head_dim=2)           # [1, 6, 2, 8]: all tokens, my heads
        ok_fwd = torch.equal(x, full[:, :, rank * 2:(rank + 1) * 2])
        back = U.gather_heads_scatter_seq(x, head_dim=2, seq_dim=1)
        ok_rt = torch.equal(back, local)
        out = U.gather_outputs_and_unpad(back.sum(-1), gather_dim=1, grad_scaler=False)  # [1, 6, 4]
        out.pow(2).sum().backward()
        expect = 2 * full.sum(-1, keepdim=True).expand_as(full)[:, rank * 3:(rank + 1) * 3]
        q.put((rank, {"fwd": ok_fwd, "rt": ok_rt, "grad": torch.allclose(local.grad, expect, atol=1e-5)}))
        dist.destroy_process_group()
    except Exception:
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))


def test_ulysses_functions_on_gloo():
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_ulysses_proc, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    for r in range(2):
        assert "error" not in res[r], res[r]["error"]
        assert res[r] == {"fwd": True, "rt": True, "grad": True}, res[r]


def test_rm_dataset_pairs(tmp_path):
    import pandas as pd

    from verl_b200.utils.dataset.rm_dataset import RMDataset

    class Tok:
        pad_token_id, eos_token_id = 0, 2

        def __call__(self, t, add_special_tokens=False):
            return {"input_ids": [ord(c) % 50 + 3 for c in t]}

    f = tmp_path / "pairs.parquet"
    pd.DataFrame({"prompt": ["hi", "yo"], "chosen": ["good", "fine"], "rejected": ["bad", "a much longer answer"]}).to_parquet(f)
    ds = RMDataset(str(f), Tok(), max_length=8)
    a, b = ds[0], ds[1]
    assert len(ds) == 2 and a["input_ids"].shape == (2, 8)
    assert a["attention_mask"].sum(-1).tolist() == [7, 6] and a["input_ids"][0, 6] == 2 and a["input_ids"][0, 7] == 0
    assert b["attention_mask"][1].sum() == 8          # truncated to max_length
    assert torch.equal(a["input_ids"][0, :2], a["input_ids"][1, :2])   # both rows start with the prompt


def test_precision_debugger_writes_per_layer_statistics(tmp_path):
    import json

    os.environ["VERL_ENGINE_DEVICE"] = "cpu"
    from verl_b200.models import get_preset
    from verl_b200.utils.profiler.precision_debugger_profile import PrecisionDebuggerProfiler
    from verl_b200.workers.config import FSDPEngineConfig, OptimizerConfig
    from verl_b200.workers.engine.native.engine import NativeEngineWithLMHead

    eng = NativeEngineWithLMHead(get_preset("tiny-llama"), FSDPEngineConfig(seed=1), OptimizerConfig(lr=1e-3))
    eng.initialize()
    ids = torch.randint(3, 500, (2, 12))
    data = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "responses": ids[:, -4:]}
    dbg = PrecisionDebuggerProfiler({"enable": True, "stages": ["actor_compute_log_prob", "nonsense"], "steps": [3]}, rank=0,
                                    save_path=str(tmp_path))
    assert not dbg.start("actor_update", 3, eng.model) and not dbg.start("actor_compute_log_prob", 2, eng.model)
    started = dbg.start("actor_compute_log_prob", 3, eng.model)
    eng.infer_batch(dict(data))
    path = dbg.stop(started)
    rows = [json.loads(l) for l in open(path)]
    L = eng.arch.num_hidden_layers
    assert [r["name"] for r in rows] == [f"layers.{i}.{k}" for i in range(L) for k in ("attn_out", "mlp_out")]
    assert all(r["nan"] == 0 and r["norm"] > 0 and r["shape"] == [24, eng.arch.hidden_size] for r in rows)
    assert eng.model.stats_hook is None


def test_clock_sampler_reads_a_fake_nvml():
    import time

    from verl_b200.utils.profiler.clocks import ClockSampler

    class FakeNvml:
        NVML_CLOCK_SM = 1

        def __init__(self):
            self.calls = 0

        def nvmlInit(self):
            pass

        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetMaxClockInfo(self, h, kind):
            return 1965

        def nvmlDeviceGetClockInfo(self, h, kind):
            self.calls += 1
            return 210 if self.calls <= 2 else 1500  # idle before the load arrives

        def nvmlDeviceGetPowerUsage(self, h):
            return 950_000

        def nvmlDeviceGetCurrentClocksEventReasons(self, h):
            return 0x4 | 0x1  # power cap + idle bit (the latter is not a throttle reason)

    s = ClockSampler(0, period_s=0.002, nvml=FakeNvml()).start()
    time.sleep(0.05)
    mid = s.snapshot()
    rec = s.stop()
    assert rec["sm_mhz"] == 1500.0 and rec["sm_max_mhz"] == 1965.0 and rec["reasons"] == ["sw_power_cap"]
    assert rec["power_w_max"] == 950.0 and rec["samples"] >= mid["samples"] > 2


def test_platform_registry_and_out_of_tree_platform(monkeypatch):
    from contextlib import contextmanager

    from verl_b200.plugin.platform import PlatformBase, PlatformRegistry, get_platform, set_platform
    from verl_b200.plugin.platform.platform_cpu import PlatformCPU
    from verl_b200.utils import device as D

    set_platform(None)
    p = get_platform()
    assert p.device_name == "cpu" and p.communication_backend_name() == "gloo" and not p.is_ipc_supported()
    assert {"b200", "cuda", "cpu"} <= set(PlatformRegistry.registered_names())
    assert D.get_nccl_backend() == "gloo" and D.get_device_id() == 0 and D.get_device_capability() == (None, None)
    b200 = PlatformRegistry.get("b200")()
    assert b200.ray_resource_options(1) == {"num_gpus": 1} and b200.visible_devices_envvar() == "CUDA_VISIBLE_DEVICES"
    assert b200.communication_backend_name() == "nccl" and b200.ray_noset_envvars()

    @PlatformRegistry.register("toy")
    class Toy(PlatformCPU):
        vendor_name = "toy"

        def communication_backend_name(self):
            return "toyccl"

        def ray_resource_name(self):
            return "TOY"

        ray_resource_options = PlatformBase.ray_resource_options

    monkeypatch.setenv("VERL_PLATFORM", "toy")
    set_platform(None)
    try:
        assert get_platform().vendor_name == "toy" and D.get_nccl_backend() == "toyccl"
        assert get_platform().ray_resource_options(2) == {"resources": {"TOY": 2}}
        with pytest.raises(AssertionError):
            PlatformRegistry.register("bad")(object)
    finally:
        monkeypatch.delenv("VERL_PLATFORM")
        set_platform(None)
    with pytest.raises(TypeError):
        PlatformBase()  # abstract


def test_tqbridge_swaps_handles_for_batches_and_writes_results_back():
    import asyncio

    from verl_b200.utils.tensordict_lite import TensorDict
    from verl_b200.utils.transfer_queue import KVBatchMeta, TransferQueue, tqbridge

    q = TransferQueue()
    for i in range(4):
        q.put(f"k{i}", {"x": torch.full((3,), float(i)), "name": f"row{i}"}, tags={"v": 0})

    class Worker:
        collects = True

        def query_collect_info(self, mesh):
            return self.collects

        @tqbridge(queue=q)
        def double(self, batch):
            assert batch.batch_size[0] == 4 and list(batch["name"]) == ["row0", "row1", "row2", "row3"]
            return TensorDict({"y": batch["x"] * 2}, batch_size=(4,))

        @tqbridge(dispatch_mode={"mesh_name": "actor"}, queue=q)
        def triple(self, batch):
            return TensorDict({"z": batch["x"] * 3}, batch_size=(len(batch["x"]),))

        @tqbridge(queue=q)
        async def norm(self, batch, scale=1.0):
            return float(batch["x"].sum()) * scale

    w = Worker()
    meta = q.get_meta(["k0", "k1", "k2", "k3"], fields=["x", "name"])
    out = w.double(meta)
    assert isinstance(out, KVBatchMeta) and out.keys == meta.keys and out.fields == ["name", "x", "y"]
    assert torch.equal(q.get(["k2"])[0]["y"], torch.full((3,), 4.0))
    # plain batches pass through untouched
    plain = w.double.__wrapped__(w, TensorDict({"x": torch.ones(4, 3), "name": ["row0", "row1", "row2", "row3"]}, batch_size=(4,)))
    assert torch.equal(plain["y"], torch.full((4, 3), 2.0))
    # only the collecting worker of a replica writes back
    w.collects = False
    assert len(w.triple(meta)) == 0 and "z" not in q.get(["k0"])[0]
    w.collects = True
    assert len(w.triple(meta)) == 4 and torch.equal(q.get(["k3"])[0]["z"], torch.full((3,), 9.0))
    # coroutine functions, and outputs that are not row batches are returned as they are
    assert asyncio.run(w.norm(meta, scale=2.0)) == pytest.approx(2.0 * 3 * (0 + 1 + 2 + 3))
