"""Batch generation through standalone rollout servers: start one replica per ``tp x dp x pp`` GPUs, spread the
prompts of a parquet/jsonl file over them (``n_samples`` per prompt), write the responses back as a new column.

Parity target: ``verl/trainer/main_generation_server.py:40-180`` (``start_server`` :40, ``generate_per_replica`` :82,
``generate`` :106, ``main`` :123). The reference talks OpenAI-style HTTP to its servers; here the replicas are
in-process handles and take token ids.
"""

from __future__ import annotations

import asyncio
import os
import sys
from typing import Optional, Sequence

import numpy as np

from ..utils.config import load_config

CONFIG_DIR = os.path.join(os.path.dirname(__file__), "config")


async def start_server(config, engines: Optional[list] = None):
    from ..workers.rollout.llm_server import LLMServerManager

    if engines is None:
        from ..workers.engine_workers import ActorRolloutRefWorker

        worker = ActorRolloutRefWorker(config=config.actor_rollout_ref, role="rollout")
        worker.init_model()
        worker.rollout.resume_kv_cache()
        engines = [worker.rollout]
    return await LLMServerManager.create(config.actor_rollout_ref.rollout, model_config=None, engines=engines)


async def generate_per_replica(client, prompts: list[list[int]], n_samples: int, sampling_params: dict, tag: str):
    async def one(i, j, ids):
        out = await client.generate(f"{tag}-{i}-{j}", prompt_ids=ids, sampling_params=dict(sampling_params))
        return i, out.token_ids

    res = await asyncio.gather(*[one(i, j, ids) for i, ids in enumerate(prompts) for j in range(n_samples)])
    grouped: list[list] = [[] for _ in prompts]
    for i, toks in res:
        grouped[i].append(toks)
    return grouped


async def generate(manager, prompts: list[list[int]], n_samples: int, sampling_params: dict):
    """Prompts are split evenly over the replicas; each replica gets its own client (sticky routing is per request)."""
    k = max(1, len(manager.replicas))
    shards = [prompts[i::k] for i in range(k)]
    outs = await asyncio.gather(*[generate_per_replica(manager.client(), sh, n_samples, sampling_params, f"gen{r}")
                                  for r, sh in enumerate(shards)])
    merged: list = [None] * len(prompts)
    for r, sh_out in enumerate(outs):
        for j, o in enumerate(sh_out):
            merged[r + j * k] = o
    return merged


def run_generation(config, tokenizer=None, engines: Optional[list] = None, prompts_ids: Optional[list[list[int]]] = None):
    import pandas as pd

    rc = config.actor_rollout_ref.rollout
    df = None
    if prompts_ids is None:
        path = os.path.expanduser(config.data.path)
        df = pd.read_json(path, lines=True) if path.endswith((".jsonl", ".json")) else pd.read_parquet(path)
        col = df[config.data.prompt_key].tolist()
        if tokenizer is None:
            from ..utils.tokenizer import hf_tokenizer

            tokenizer = hf_tokenizer(config.actor_rollout_ref.model.path)
        prompts_ids = [tokenizer.apply_chat_template(list(c), add_generation_prompt=True, tokenize=True) if not isinstance(c, str)
                       else tokenizer.encode(c) for c in col]
    sp = dict(temperature=float(rc.temperature), top_p=float(rc.top_p), top_k=int(rc.top_k), max_tokens=int(rc.response_length), logprobs=False)

    async def go():
        mgr = await start_server(config, engines)
        return await generate(mgr, prompts_ids, int(config.data.n_samples), sp)

    outs = asyncio.run(go())
    if df is not None:
        df["responses"] = [[tokenizer.decode(t, skip_special_tokens=True) for t in group] for group in outs]
        out_path = os.path.expanduser(config.data.output_path)
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        df.to_parquet(out_path)
    return outs


def main(argv: Optional[Sequence[str]] = None):
    argv = list(sys.argv[1:] if argv is None else argv)
    return run_generation(load_config(CONFIG_DIR, "generation", argv))


if __name__ == "__main__":
    main()
