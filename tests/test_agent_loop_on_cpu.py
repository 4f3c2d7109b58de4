"""Agent loops against real in-process rollout engines (tiny CPU model): single turn, tool calls, load balancing."""
import asyncio

import numpy as np
import torch

from verl_b200 import DataProto
from verl_b200.experimental.agent_loop import AgentLoopManager
from verl_b200.experimental.agent_loop.tool_agent_loop import ToolAgentLoop
from verl_b200.experimental.agent_loop.tool_parser import ToolParser
from verl_b200.models import FlatParams, get_preset
from verl_b200.tools import FunctionTool
from verl_b200.utils.config import DictConfig
from verl_b200.workers.rollout.llm_server import FullyAsyncLLMServerClient, GlobalRequestLoadBalancer, LLMServerManager
from verl_b200.workers.rollout.native.engine import RolloutEngine
from verl_b200.workers.rollout.replica import TokenOutput


def _cfg(P=8, R=12):
    return DictConfig({"actor_rollout_ref": {"rollout": {"name": "native", "prompt_length": P, "response_length": R, "temperature": 1.0,
                                                         "top_p": 1.0, "top_k": -1, "do_sample": True, "calculate_log_probs": True,
                                                         "tensor_model_parallel_size": 1, "agent": {"num_workers": 2},
                                                         "val_kwargs": {"temperature": 0.0, "do_sample": False},
                                                         "multi_turn": {"format": "hermes", "max_parallel_calls": 2,
                                                                        "max_tool_response_length": 32}}}})


def _engines(n=2):
    cfg = get_preset("tiny-qwen2")
    P = FlatParams(cfg, dtype=torch.float32)
    P.init_weights(seed=3, std=0.1)
    return [RolloutEngine(cfg, P, max_num_seqs=4, max_model_len=64, block_size=8, sync_interval=2, eos_token_id=-1) for _ in range(n)]


def test_single_turn_manager_layout():
    config = _cfg()
    rc = config.actor_rollout_ref.rollout

    async def go():
        mgr = await LLMServerManager.create(rc, engines=_engines(2), model_config=None)
        alm = AgentLoopManager(config, mgr)
        ids = torch.randint(3, 500, (6, 8))
        am = torch.ones(6, 8, dtype=torch.int64)
        am[0, :3] = 0  # left padding
        batch = DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": am}, meta_info={"temperature": 1.0})
        out = await alm.generate_sequences_async(batch)
        return ids, am, out, mgr

    ids, am, out, mgr = asyncio.run(go())
    assert out.batch["responses"].shape == (6, 12) and out.batch["input_ids"].shape == (6, 20)
    assert torch.equal(out.batch["prompts"][1], ids[1]) and out.batch["attention_mask"][0, :3].sum() == 0
    assert out.batch["response_mask"].sum(-1).tolist() == [12] * 6
    assert (out.batch["rollout_log_probs"] <= 0).all() and out.batch["position_ids"][0, 3] == 0
    assert out.non_tensor_batch["__num_turns__"].tolist() == [2] * 6
    assert sum(mgr.lb.snapshot().values()) == 0  # every acquired server was released


def test_tool_loop_masks_tool_tokens():
    config = _cfg(P=8, R=200)

    class ScriptedServer:
        """First turn emits a hermes tool call, second turn a plain answer."""

        def __init__(self):
            self.calls = 0

        async def generate(self, request_id, prompt_ids, sampling_params, **kw):
            self.calls += 1
            text = '<tool_call>{"name": "add", "arguments": {"a": 2, "b": 3}}</tool_call>' if self.calls == 1 else "done"
            return TokenOutput(token_ids=[ord(c) for c in text], log_probs=[-0.1] * len(text), stop_reason="completed")

    class CharTok:
        pad_token_id = 0
        chat_template = None

        def decode(self, ids, **kw):
            return "".join(chr(i) for i in ids)

        def apply_chat_template(self, messages, tools=None, add_generation_prompt=True, tokenize=True, **kw):
            text = "".join(f"<{m['role']}>{m['content']}" for m in messages) + ("<assistant>" if add_generation_prompt else "")
            return [ord(c) for c in text]

    def add(a: int, b: int) -> int:
        """Add two integers."""
        return a + b

    srv = ScriptedServer()
    loop = ToolAgentLoop(config, srv, tokenizer=CharTok(), tools=[FunctionTool(add)])
    out = asyncio.run(loop.run({"temperature": 1.0}, raw_prompt_ids=[5, 6, 7]))
    text = "".join(chr(i) for i in out.response_ids)
    assert srv.calls == 2 and "5" in text and text.endswith("done")
    n_call = len('<tool_call>{"name": "add", "arguments": {"a": 2, "b": 3}}</tool_call>')
    assert out.response_mask[:n_call] == [1] * n_call and 0 in out.response_mask and out.response_mask[-4:] == [1] * 4
    assert out.num_turns == 4 and len(out.response_ids) == len(out.response_mask) == len(out.response_logprobs)


def test_tool_parsers():
    async def go(name, text):
        return await ToolParser.get_tool_parser(name).extract_tool_calls([], text=text)

    c, calls = asyncio.run(go("hermes", 'hi <tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call> bye'))
    assert calls[0].name == "f" and '"x": 1' in calls[0].arguments and "tool_call" not in c
    _, calls = asyncio.run(go("qwen3_xml", "<tool_call><function=g><parameter=k>7</parameter></function></tool_call>"))
    assert calls[0].name == "g" and calls[0].arguments == '{"k": 7}'
    _, calls = asyncio.run(go("gpt-oss", '<|channel|>commentary to=functions.h <|constrain|>json<|message|>{"q": "a"}<|call|>'))
    assert calls[0].name == "h"
    _, calls = asyncio.run(go("llama3_json", '<|python_tag|>{"name": "z", "parameters": {"p": 2}}'))
    assert calls[0].name == "z"


def test_load_balancer_sticky_least_loaded_and_elastic():
    lb = GlobalRequestLoadBalancer(["a", "b"])
    s1 = lb.acquire_server("r1")
    s2 = lb.acquire_server("r2")
    assert {s1, s2} == {"a", "b"} and lb.acquire_server("r1") == s1  # sticky
    lb.release_server(s1)
    lb.release_server(s1)
    lb.add_servers(["c"])
    assert lb.acquire_server("r3") in ("c", s1)
    lb.remove_servers([s1])
    assert lb.acquire_server("r1") != s1
    empty = GlobalRequestLoadBalancer([])
    assert empty.acquire_server("x") is None


def test_fully_async_client_resumes_after_abort():
    class Flaky:
        def __init__(self):
            self.n = 0

        async def generate(self, prompt_ids, sampling_params, request_id, **kw):
            self.n += 1
            if self.n == 1:
                return TokenOutput([1, 2], [-0.1, -0.2], stop_reason="aborted")
            assert prompt_ids[-2:] == [1, 2] and sampling_params["max_tokens"] == 4
            return TokenOutput([3, 4, 5, 6], [-0.3] * 4, stop_reason="length")

    cfg = DictConfig({"prompt_length": 4, "response_length": 6})
    cl = FullyAsyncLLMServerClient(cfg, {"s": Flaky()}, GlobalRequestLoadBalancer(["s"]), retry_interval=0.0)
    out = asyncio.run(cl.generate("req", prompt_ids=[9, 9], sampling_params={"max_tokens": 6}))
    assert out.token_ids == [1, 2, 3, 4, 5, 6] and len(out.log_probs) == 6 and out.stop_reason == "length"


def test_trajectory_info_greedy_rows_traces_and_performance_metrics():
    """Rows of one dataset index get consecutive repeat numbers; a row marked ``__do_sample__ = False`` is decoded greedily
    while its neighbours sample; traced spans carry the trajectory of the task that recorded them (the trajectories run
    concurrently); the manager reports min / max / mean of every timer and the slowest trajectory."""
    from verl_b200.experimental.agent_loop.agent_loop import get_trajectory_info
    from verl_b200.utils.rollout_trace import TRACE_RING, RolloutTraceConfig

    info = get_trajectory_info(7, [4, 4, 4, 9, 9, 2], False)
    assert [t["rollout_n"] for t in info] == [0, 1, 2, 0, 1, 0] and info[3] == {"step": 7, "sample_index": 9, "rollout_n": 0, "validate": False}

    config = _cfg()
    rc = config.actor_rollout_ref.rollout
    RolloutTraceConfig.init("p", "e", "memory", max_samples_per_step_per_worker=1)
    TRACE_RING.clear()

    class Scorer:
        async def compute_score_for(self, out, kwargs):
            await asyncio.sleep(0.01)
            return float(len(out.response_ids))

    async def go(greedy_rows):
        mgr = await LLMServerManager.create(rc, engines=_engines(1), model_config=None)
        alm = AgentLoopManager(config, mgr, num_workers=1, reward_loop_worker=Scorer())
        g = torch.Generator().manual_seed(0)
        row = torch.randint(3, 500, (1, 8), generator=g)
        ids = row.repeat(4, 1)                                      # four repeats of two dataset rows
        batch = DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": torch.ones(4, 8, dtype=torch.int64)},
                                    non_tensors={"index": np.array([11, 11, 12, 12]),
                                                 "__do_sample__": np.array([i not in greedy_rows for i in range(4)])},
                                    meta_info={"temperature": 1.0, "global_steps": 3})
        return await alm.generate_sequences_async(batch)

    out = asyncio.run(go({1, 3}))
    resp = out.batch["responses"]
    assert torch.equal(resp[1], resp[3])                             # same prompt, both greedy
    assert not torch.equal(resp[0], resp[1]) or not torch.equal(resp[2], resp[3])   # the sampled rows differ from the greedy ones
    assert out.batch["rm_scores"].sum(-1).tolist() == [12.0] * 4
    t = out.meta_info["timing"]
    for k in ("generate_sequences", "tool_calls", "compute_score", "num_preempted"):
        assert t[f"agent_loop/{k}/min"] <= t[f"agent_loop/{k}/mean"] <= t[f"agent_loop/{k}/max"]
    assert t["agent_loop/compute_score/min"] >= 0.01 and t["agent_loop/slowest/prompt_length"] == 8 and t["agent_loop/slowest/response_length"] == 12
    spans = [s for s in TRACE_RING if s["op"].endswith("_run_traced")]
    assert len(spans) == 2 and len({s["sample_index"] for s in spans}) == 1      # one dataset row traced: both of its repeats
    assert sorted(s["rollout_n"] for s in spans) == [0, 1] and all(s["step"] == 3 for s in spans)
    RolloutTraceConfig.reset()


def test_expert_choices_of_the_rollout_land_on_the_padded_positions():
    """Router replay from the rollout: per-trajectory records [tokens, layers, top-k] are placed on the padded
    [prompt | response] positions; a trajectory without a record keeps zeros; a truncated prompt drops leading positions."""
    from verl_b200.experimental.agent_loop.agent_loop import AgentLoopOutput, AgentLoopWorker

    config = _cfg(P=4, R=3)
    w = AgentLoopWorker(config, server_manager=None)

    def rec(n_pos, base):
        return (torch.arange(n_pos * 2 * 2).reshape(n_pos, 2, 2) + base).to(torch.int32)

    outs = [AgentLoopOutput(prompt_ids=[5, 6], response_ids=[7, 8, 9], response_mask=[1, 1, 1], routed_experts=rec(4, 100)),
            AgentLoopOutput(prompt_ids=[1, 2, 3, 4, 5, 6], response_ids=[7], response_mask=[1], routed_experts=rec(6, 200)),
            AgentLoopOutput(prompt_ids=[5], response_ids=[7, 8], response_mask=[1, 1])]
    out = w._postprocess(outs, DataProto(meta_info={"pad_token_id": 0}))
    r = out.batch["routed_experts"]
    assert r.shape == (3, 7, 2, 2) and r.dtype == torch.int32
    # row 0: two prompt tokens sit at positions 2..3, responses from 4; four recorded positions (the last generated token never
    # went through the rollout model)
    assert torch.equal(r[0, 2:6], rec(4, 100)) and int(r[0, :2].abs().sum()) == 0 and int(r[0, 6].abs().sum()) == 0
    # row 1: the prompt was cut to its last four tokens, so the first two recorded positions go with it
    assert torch.equal(out.batch["prompts"][1], torch.tensor([3, 4, 5, 6])) and torch.equal(r[1, 0:4], rec(6, 200)[2:6])
    assert int(r[2].abs().sum()) == 0
    assert "routed_experts" not in w._postprocess(outs[2:], DataProto(meta_info={"pad_token_id": 0})).batch.keys()


from verl_b200.experimental.agent_loop.single_turn_agent_loop import SingleTurnAgentLoop  # noqa: E402


class PrefixedLoop(SingleTurnAgentLoop):
    """Declared through a configuration file below; defined at module level so the dotted path resolves."""

    def __init__(self, *a, marker=None, **k):
        super().__init__(*a, **k)
        self.marker = marker

    async def run(self, sampling_params, **kwargs):
        out = await super().run(sampling_params, **kwargs)
        out.extra_fields["marker"] = self.marker
        return out


def test_agent_loops_declared_in_a_configuration_file(tmp_path, monkeypatch):
    from verl_b200.experimental.agent_loop import agent_loop as al
    from verl_b200.experimental.agent_loop.utils import (build_gpt_oss_tool_response_text, load_agent_loop_configs,
                                                         resolve_config_path)

    (tmp_path / "loops.yaml").write_text("- name: prefixed\n  _target_: tests.test_agent_loop_on_cpu.PrefixedLoop\n  marker: 7\n")
    monkeypatch.chdir(tmp_path)
    assert resolve_config_path("loops.yaml") == str(tmp_path / "loops.yaml")
    assert load_agent_loop_configs("loops.yaml")["prefixed"][1] == {"marker": 7}
    import pytest

    with pytest.raises(FileNotFoundError):
        resolve_config_path("../outside.yaml")
    config = _cfg()
    config.actor_rollout_ref.rollout.agent["agent_loop_config_path"] = "loops.yaml"
    config.actor_rollout_ref.rollout.agent["default_agent_loop"] = "prefixed"

    async def go():
        mgr = await LLMServerManager.create(config.actor_rollout_ref.rollout, engines=_engines(1), model_config=None)
        alm = AgentLoopManager(config, mgr)
        ids = torch.randint(3, 500, (2, 8))
        return await alm.generate_sequences_async(DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": torch.ones(2, 8, dtype=torch.int64)},
                                                                      meta_info={"temperature": 1.0}))

    out = asyncio.run(go())
    assert out.non_tensor_batch["marker"].tolist() == [7, 7] and al._AGENT_LOOP_KWARGS["prefixed"] == {"marker": 7}
    text = build_gpt_oss_tool_response_text([{"content": "4"}, {"content": "ok"}], ["add", "ping"])
    assert text == ("<|start|>functions.add to=assistant<|channel|>commentary<|message|>4<|end|>"
                    "<|start|>functions.ping to=assistant<|channel|>commentary<|message|>ok<|end|><|start|>assistant")
