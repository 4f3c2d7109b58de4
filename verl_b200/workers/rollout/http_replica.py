"""Replicas backed by an inference server that runs somewhere else and is reached over HTTP: an SGLang server (native
``/generate`` API) or any OpenAI-compatible completion server (vLLM's ``vllm serve``, TensorRT-LLM's ``trtllm-serve``).

The framework's own engine lives in the trainer's process and needs none of this; these replicas exist for deployments
that already operate such servers (standalone rollout pools, reward-model servers). Token ids go in, token ids and their
log-probs come back, so no tokenizer round trip changes the sequence. Weight updates go through a checkpoint directory the
server can read (``update_weights_from_path``); memory hand-back, cache flush and abort map to the servers' control
endpoints where they have one and are no-ops otherwise.

Parity target: the server adapters of ``verl/workers/rollout/sglang_rollout/http_server_engine.py`` (generate :640-720,
``update_weights_from_tensor`` / ``flush_cache`` / ``release_memory_occupation`` / ``resume_memory_occupation`` /
``abort_request``), ``verl/workers/rollout/trtllm_rollout/trtllm_async_server.py`` and the replica registry of
``verl/workers/rollout/replica.py:302-408``.
"""

from __future__ import annotations

import asyncio
from typing import Any, Optional

from .replica import RolloutReplica, TokenOutput

__all__ = ["HTTPInferenceServer", "HTTPReplica", "OpenAIReplica"]


class HTTPInferenceServer:
    """Client side of one remote server. ``dialect``: ``sglang`` | ``openai``."""

    def __init__(self, base_url: str, dialect: str = "sglang", model: Optional[str] = None, timeout: float = 600.0,
                 max_retries: int = 3, retry_delay: float = 0.5, api_key: Optional[str] = None):
        assert dialect in ("sglang", "openai"), f"unknown server dialect {dialect!r}"
        self.base, self.dialect, self.model = base_url.rstrip("/"), dialect, model or "default"
        self.timeout, self.max_retries, self.retry_delay = float(timeout), int(max_retries), float(retry_delay)
        self.headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
        self._session = None
        self._global_steps = 0

    # ------------------------------------------------------------------ transport
    async def _http(self, method: str, path: str, payload: Optional[dict] = None, params: Optional[dict] = None, ok_missing: bool = False):
        import aiohttp

        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout), headers=self.headers)
        last: Optional[BaseException] = None
        for attempt in range(self.max_retries + 1):
            try:
                async with self._session.request(method, self.base + path, json=payload, params=params) as r:
                    if r.status == 404 and ok_missing:
                        return None       # this server has no such control endpoint
                    if r.status >= 500:
                        raise RuntimeError(f"{path}: HTTP {r.status}: {(await r.text())[:200]}")
                    if r.status >= 400:
                        raise ValueError(f"{path}: HTTP {r.status}: {(await r.text())[:200]}")   # the request itself is wrong: no retry
                    if "json" in (r.headers.get("Content-Type") or ""):
                        return await r.json()
                    return await r.text()
            except ValueError:
                raise
            except (aiohttp.ClientError, asyncio.TimeoutError, RuntimeError) as e:   # connection trouble and 5xx are retried
                last = e
                if attempt < self.max_retries:
                    await asyncio.sleep(self.retry_delay * (2 ** attempt))
        raise ConnectionError(f"{self.base}{path} failed after {self.max_retries + 1} attempts: {last!r}")

    async def close(self) -> None:
        if self._session is not None and not self._session.closed:
            await self._session.close()

    # ------------------------------------------------------------------ generation
    async def generate(self, prompt_ids: list[int], sampling_params: dict, request_id: str, **kwargs) -> TokenOutput:
        sp = dict(sampling_params or {})
        max_tokens = sp.pop("max_tokens", sp.pop("max_new_tokens", None))
        want_lp = bool(sp.pop("logprobs", True))
        if self.dialect == "sglang":
            body_sp = {k: sp[k] for k in ("temperature", "top_p", "top_k", "repetition_penalty", "stop_token_ids", "ignore_eos") if k in sp}
            if max_tokens is not None:
                body_sp["max_new_tokens"] = int(max_tokens)
            res = await self._http("POST", "/generate", {"rid": request_id, "input_ids": list(map(int, prompt_ids)),
                                                         "sampling_params": body_sp, "return_logprob": want_lp})
            meta = res.get("meta_info", {})
            lps = meta.get("output_token_logprobs") or []
            toks = res.get("output_ids") or [int(t[1]) for t in lps]
            fin = (meta.get("finish_reason") or {})
            kind = fin.get("type") if isinstance(fin, dict) else fin
            reason = {"stop": "completed", "length": "length", "abort": "aborted"}.get(kind, kind)
            return TokenOutput(token_ids=list(map(int, toks)), log_probs=[float(t[0]) for t in lps] if want_lp and lps else None,
                               stop_reason=reason, extra_fields={"global_steps": self._global_steps})
        body = {"model": self.model, "prompt": list(map(int, prompt_ids)), "max_tokens": int(max_tokens) if max_tokens is not None else 16,
                "temperature": float(sp.get("temperature", 1.0)), "top_p": float(sp.get("top_p", 1.0)),
                "logprobs": 0 if want_lp else None, "return_tokens_as_token_ids": True}
        if int(sp.get("top_k", -1) or -1) > 0:
            body["top_k"] = int(sp["top_k"])
        if sp.get("seed") is not None:
            body["seed"] = int(sp["seed"])
        res = await self._http("POST", "/v1/completions", {k: v for k, v in body.items() if v is not None})
        ch = res["choices"][0]
        lp = ch.get("logprobs") or {}
        toks = [int(str(t).split(":")[-1]) for t in (lp.get("tokens") or [])]     # "token_id:123"
        if not toks and ch.get("token_ids") is not None:
            toks = list(map(int, ch["token_ids"]))
        reason = {"stop": "completed", "length": "length", "abort": "aborted"}.get(ch.get("finish_reason"), ch.get("finish_reason"))
        return TokenOutput(token_ids=toks, log_probs=[float(x) for x in lp.get("token_logprobs") or []] if want_lp else None,
                           stop_reason=reason, extra_fields={"global_steps": self._global_steps})

    # ------------------------------------------------------------------ control
    async def healthy(self) -> bool:
        try:
            await self._http("GET", "/health" if self.dialect == "openai" else "/health_generate", ok_missing=True)
            return True
        except (ConnectionError, ValueError):
            return False

    async def wake_up(self):
        if self.dialect == "sglang":
            await self._http("POST", "/resume_memory_occupation", {}, ok_missing=True)
        else:
            await self._http("POST", "/wake_up", ok_missing=True)

    async def sleep(self):
        if self.dialect == "sglang":
            await self._http("POST", "/release_memory_occupation", {}, ok_missing=True)
        else:
            await self._http("POST", "/sleep", params={"level": "1"}, ok_missing=True)

    async def clear_kv_cache(self):
        if self.dialect == "sglang":
            await self._http("POST", "/flush_cache", ok_missing=True)
        else:
            await self._http("POST", "/reset_prefix_cache", ok_missing=True)

    async def abort_all_requests(self):
        if self.dialect == "sglang":
            await self._http("POST", "/abort_request", {"abort_all": True}, ok_missing=True)

    async def resume_generation(self):
        return None

    async def set_global_steps(self, steps: int):
        self._global_steps = int(steps)

    async def update_weights_from_path(self, path: str) -> Any:
        """Make the server load the HF checkpoint at ``path`` (a directory both sides can read)."""
        if self.dialect == "sglang":
            res = await self._http("POST", "/update_weights_from_disk", {"model_path": str(path)})
            if isinstance(res, dict) and res.get("success") is False:
                raise RuntimeError(f"weight update refused: {res.get('message')}")
            return res
        # OpenAI-compatible servers have no standard reload call; vLLM's development endpoint is tried, absence is an error
        res = await self._http("POST", "/collective_rpc", {"method": "reload_weights", "kwargs": {"model_path": str(path)}}, ok_missing=True)
        if res is None:
            raise NotImplementedError("this server exposes no weight reload endpoint; restart it on the new checkpoint")
        return res


class HTTPReplica(RolloutReplica):
    """One replica per server URL (``rollout.server_urls``; replica ``i`` takes URL ``i``)."""

    dialect = "sglang"

    def __init__(self, replica_rank, config, model_config, gpus_per_node: int = 8, is_reward_model: bool = False, url: Optional[str] = None):
        super().__init__(replica_rank, config, model_config, gpus_per_node, is_reward_model)
        g = config.get if hasattr(config, "get") else lambda k, d=None: getattr(config, k, d)
        urls = list(g("server_urls", None) or [])
        self.url = url or (urls[replica_rank % len(urls)] if urls else None)
        self._opts = dict(dialect=g("server_dialect", None) or self.dialect, model=g("served_model_name", None),
                          timeout=float(g("server_timeout", 600.0) or 600.0), api_key=g("server_api_key", None))

    async def launch_servers(self):
        assert self.url, "rollout.server_urls is empty: an HTTP replica connects to a server that is already running"
        srv = HTTPInferenceServer(self.url, **self._opts)
        self.servers = [srv]
        self._server_handle = srv
        self._server_address = self.url

    async def update_weights(self, params, directory: str) -> None:
        """Write the working weights as an HF checkpoint into ``directory`` and make the server load it."""
        from ...utils.model import save_hf_weights

        save_hf_weights(params, directory)
        params.cfg.save_pretrained(directory)
        await self.servers[0].update_weights_from_path(directory)


class OpenAIReplica(HTTPReplica):
    dialect = "openai"
