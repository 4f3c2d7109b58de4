"""Optional adapter that serves ``generate_sequences`` through an installed vLLM instead of the native rollout engine
(``rollout.name=vllm``): for users who need a model family or a sampling feature the native engine does not cover. The
native engine is the default and the measured path; this adapter is a library call and is only exercised where vLLM and a
GPU are present.

Token-in / token-out: left-padded prompt ids go in as ``prompt_token_ids``, responses come back as ids with their
sampled-token log-probs and are right-padded to ``response_length``. ``update_weights`` streams (name, tensor) pairs in
the HuggingFace layout into the engine's model; ``release`` / ``resume`` map to vLLM's sleep / wake-up.

Parity target: ``verl/workers/rollout/vllm_rollout/vllm_rollout.py`` (``ServerAdapter``: ``resume/release`` :194-206,
``update_weights`` :208-246) and ``vllm_async_server.py`` (``generate`` :535-720).
"""

from __future__ import annotations

from typing import Generator

import torch

from ....protocol import DataProto
from ....utils.tensordict_lite import TensorDict
from ..base import BaseRollout

__all__ = ["VLLMRollout"]


def _cfg(config, key, default=None):
    return config.get(key, default) if hasattr(config, "get") else getattr(config, key, default)


class VLLMRollout(BaseRollout):
    def __init__(self, config, model_config, device_mesh=None):
        super().__init__(config, model_config, device_mesh)
        try:
            from vllm import LLM
        except Exception as e:  # not installed, or no usable device
            raise ImportError(f"rollout.name=vllm needs an importable vLLM ({type(e).__name__}: {e}); "
                              f"use rollout.name=native for the built-in engine") from e
        path = _cfg(model_config, "local_path", None) or _cfg(model_config, "path")
        max_len = int(_cfg(config, "max_model_len", None) or (_cfg(config, "prompt_length") + _cfg(config, "response_length")))
        self.llm = LLM(model=path, skip_tokenizer_init=True, tensor_parallel_size=int(_cfg(config, "tensor_model_parallel_size", 1) or 1),
                       dtype=str(_cfg(config, "dtype", "bfloat16")), enforce_eager=bool(_cfg(config, "enforce_eager", False)),
                       gpu_memory_utilization=float(_cfg(config, "gpu_memory_utilization", 0.5)), max_model_len=max_len,
                       max_num_seqs=int(_cfg(config, "max_num_seqs", 256)), enable_sleep_mode=bool(_cfg(config, "free_cache_engine", True)),
                       load_format=str(_cfg(config, "load_format", "auto")), seed=int(_cfg(config, "seed", 0) or 0))

    # ---- memory hand-over with a colocated trainer
    async def resume(self, tags: list[str]):
        self.llm.wake_up(tags=tags)

    async def release(self):
        self.llm.sleep(level=1)

    async def update_weights(self, weights: Generator[tuple[str, torch.Tensor], None, None], **kwargs):
        def load(worker_self, pairs):
            worker_self.model_runner.model.load_weights(pairs)

        self.llm.collective_rpc(load, args=(list(weights),))
        self.llm.reset_prefix_cache()

    # ---- generation
    @torch.no_grad()
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        from vllm import SamplingParams

        mi = prompts.meta_info
        ids, am = prompts.batch["input_ids"], prompts.batch["attention_mask"]
        b, P = ids.shape
        R = int(_cfg(self.config, "response_length"))
        greedy = not mi.get("do_sample", _cfg(self.config, "do_sample", True))
        n = 1 if greedy or mi.get("validate", False) else int(mi.get("n", _cfg(self.config, "n", 1)) or 1)
        sp = SamplingParams(n=n, max_tokens=R, logprobs=0, detokenize=False,
                            temperature=0.0 if greedy else float(mi.get("temperature", _cfg(self.config, "temperature", 1.0))),
                            top_p=float(mi.get("top_p", _cfg(self.config, "top_p", 1.0))),
                            top_k=int(mi.get("top_k", _cfg(self.config, "top_k", -1)) or -1))
        reqs = [{"prompt_token_ids": ids[i][am[i].bool()].tolist()} for i in range(b)]
        outs = self.llm.generate(reqs, sampling_params=sp, use_tqdm=False)
        pad = mi.get("pad_token_id", _cfg(self.model_config, "pad_token_id", 0)) or 0
        resp = torch.full((b * n, R), pad, dtype=ids.dtype)
        lps = torch.zeros(b * n, R, dtype=torch.float32)
        rmask = torch.zeros(b * n, R, dtype=am.dtype)
        for i, o in enumerate(outs):
            for j, c in enumerate(o.outputs):
                t = list(c.token_ids)[:R]
                row = i * n + j
                resp[row, : len(t)] = torch.tensor(t, dtype=ids.dtype)
                rmask[row, : len(t)] = 1
                if c.logprobs:
                    lps[row, : len(t)] = torch.tensor([c.logprobs[k][t[k]].logprob for k in range(len(t))])
        dev = ids.device
        ids_n, am_n = ids.repeat_interleave(n, 0), am.repeat_interleave(n, 0)
        seq = torch.cat([ids_n, resp.to(dev)], 1)
        mask = torch.cat([am_n, rmask.to(dev)], 1)
        pos = (torch.cumsum(mask, -1) - 1).clamp_min(0)
        batch = TensorDict({"prompts": ids_n, "responses": resp.to(dev), "input_ids": seq, "attention_mask": mask, "position_ids": pos,
                            "response_mask": rmask.to(dev), "rollout_log_probs": lps.to(dev)}, batch_size=b * n)
        return DataProto(batch=batch, meta_info=dict(mi))
