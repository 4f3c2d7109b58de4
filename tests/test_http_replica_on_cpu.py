"""Replicas that talk to an inference server over HTTP, against in-process fake servers of both dialects."""
import asyncio

import pytest
import torch

aiohttp = pytest.importorskip("aiohttp")
from aiohttp import web  # noqa: E402

from verl_b200.utils.config import DictConfig  # noqa: E402
from verl_b200.workers.rollout.llm_server import LLMServerManager  # noqa: E402
from verl_b200.workers.rollout.replica import get_rollout_replica_class  # noqa: E402


class _Fake:
    """Echo model: the n-th generated token is (last prompt token + n) % 1000, log-prob -0.1 * n."""

    def __init__(self, dialect):
        self.dialect, self.calls, self.fail_first = dialect, [], 0
        app = web.Application()
        if dialect == "sglang":
            app.router.add_post("/generate", self.sglang_generate)
            for path in ("/flush_cache", "/release_memory_occupation", "/resume_memory_occupation", "/abort_request",
                         "/update_weights_from_disk"):
                app.router.add_post(path, self.control)
        else:
            app.router.add_post("/v1/completions", self.openai_generate)
            app.router.add_post("/sleep", self.control)
        self.app = app

    async def control(self, req):
        body = await req.json() if req.can_read_body else {}
        self.calls.append((req.path, body))
        return web.json_response({"success": True})

    async def sglang_generate(self, req):
        if self.fail_first > 0:
            self.fail_first -= 1
            return web.Response(status=503, text="busy")
        b = await req.json()
        self.calls.append(("/generate", b))
        n = b["sampling_params"]["max_new_tokens"]
        toks = [(b["input_ids"][-1] + i + 1) % 1000 for i in range(n)]
        return web.json_response({"output_ids": toks, "meta_info": {"finish_reason": {"type": "length"},
                                                                  "output_token_logprobs": [[-0.1 * (i + 1), t, None] for i, t in enumerate(toks)]}})

    async def openai_generate(self, req):
        b = await req.json()
        self.calls.append(("/v1/completions", b))
        if not isinstance(b["prompt"], list) or b["max_tokens"] > 64:
            return web.Response(status=400, text="bad request")
        toks = [(b["prompt"][-1] + i + 1) % 1000 for i in range(b["max_tokens"])]
        return web.json_response({"choices": [{"finish_reason": "stop", "logprobs": {"tokens": [f"token_id:{t}" for t in toks],
                                                                                     "token_logprobs": [-0.1 * (i + 1) for i in range(len(toks))]}}]})


async def _serve(fake):
    runner = web.AppRunner(fake.app)
    await runner.setup()
    site = web.TCPSite(runner, "127.0.0.1", 0)
    await site.start()
    port = site._server.sockets[0].getsockname()[1]
    return runner, f"http://127.0.0.1:{port}"


def test_sglang_dialect_generate_control_retry_and_weight_update(tmp_path):
    async def go():
        fake = _Fake("sglang")
        runner, url = await _serve(fake)
        try:
            rc = DictConfig({"name": "sglang", "server_urls": [url], "prompt_length": 8, "response_length": 5, "server_timeout": 10})
            mgr = await LLMServerManager.create(rc)
            assert list(mgr.servers) == [url]
            client = mgr.client()
            fake.fail_first = 2                                      # two 503 answers, then success
            mgr.replicas[0].servers[0].retry_delay = 0.01
            out = await client.generate("r0", prompt_ids=[5, 6, 7], sampling_params={"temperature": 0.7, "top_k": 20, "max_tokens": 4})
            assert out.token_ids == [8, 9, 10, 11] and out.stop_reason == "length"
            assert out.log_probs == pytest.approx([-0.1, -0.2, -0.3, -0.4])
            sent = [c for c in fake.calls if c[0] == "/generate"][-1][1]
            assert sent["input_ids"] == [5, 6, 7] and sent["return_logprob"] and sent["sampling_params"]["top_k"] == 20
            await mgr.sleep()
            await mgr.wake_up()
            await mgr.clear_kv_cache()
            paths = [c[0] for c in fake.calls]
            assert "/release_memory_occupation" in paths and "/resume_memory_occupation" in paths and "/flush_cache" in paths
            # weights: an HF checkpoint directory is written and the server is told to load it
            from verl_b200.models import FlatParams, get_preset

            P = FlatParams(get_preset("tiny-qwen2"), dtype=torch.float32)
            P.init_weights(seed=0)
            await mgr.replicas[0].update_weights(P, str(tmp_path / "ckpt"))
            assert (tmp_path / "ckpt" / "config.json").exists()
            assert fake.calls[-1] == ("/update_weights_from_disk", {"model_path": str(tmp_path / "ckpt")})
            await mgr.replicas[0].servers[0].close()
        finally:
            await runner.cleanup()

    asyncio.run(go())


def test_openai_dialect_and_error_handling():
    async def go():
        fake = _Fake("openai")
        runner, url = await _serve(fake)
        try:
            cls = get_rollout_replica_class("trtllm")
            rep = cls(0, DictConfig({"server_urls": [url], "served_model_name": "policy"}), None)
            await rep.init_standalone()
            srv = rep.servers[0]
            out = await srv.generate([1, 2, 3], {"temperature": 0.0, "max_tokens": 3, "seed": 4}, "r1")
            assert out.token_ids == [4, 5, 6] and out.stop_reason == "completed" and out.log_probs == pytest.approx([-0.1, -0.2, -0.3])
            sent = fake.calls[-1][1]
            assert sent["model"] == "policy" and sent["prompt"] == [1, 2, 3] and sent["return_tokens_as_token_ids"] and sent["seed"] == 4
            with pytest.raises(ValueError, match="400"):            # a malformed request is not retried
                await srv.generate([1], {"max_tokens": 100}, "r2")
            await rep.sleep()                                        # the fake knows /sleep
            await rep.clear_kv_cache()                               # ... but no /reset_prefix_cache: a no-op
            with pytest.raises(NotImplementedError):
                await srv.update_weights_from_path("/nowhere")
            await srv.close()
        finally:
            await runner.cleanup()
        dead = get_rollout_replica_class("openai")(0, DictConfig({"server_urls": ["http://127.0.0.1:9"]}), None)
        await dead.init_standalone()
        dead.servers[0].max_retries, dead.servers[0].retry_delay = 1, 0.01
        assert not await dead.servers[0].healthy()
        await dead.servers[0].close()

    asyncio.run(go())
