"""Prefill / decode disaggregation: prompts are prefilled by one engine (replica, GPU) and decoded by another; the
prompt's KV pages, the first sampled token and the sampler state travel between them. Long prefills then never stall the
decode batches of other requests, and the two stages can be sized independently.

Both engines serve the same model with the same KV block size; on GPUs the KV hand-off is a peer copy over NVLink.
Parity target: ``verl/workers/rollout/vllm_rollout/vllm_pd_replica.py`` / ``sglang_rollout/sglang_pd_replica.py``
(prefill and decode replicas with KV transfer) and ``verl/workers/config/disaggregation.py``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

from .native.engine import RequestOutput, RolloutEngine, SamplingParams

__all__ = ["DisaggregationConfig", "PrefillDecodeRollout"]


@dataclass
class DisaggregationConfig:
    enable: bool = False
    prefill_replicas: int = 1
    decode_replicas: int = 1
    prefill_chunk: int = 0      # prompts handed over per round (0 = as many as the prefill engine admits)


class PrefillDecodeRollout:
    """``generate`` with the same contract as ``RolloutEngine.generate`` over a prefill engine and a decode engine."""

    def __init__(self, prefill: RolloutEngine, decode: RolloutEngine, config: Optional[DisaggregationConfig] = None):
        assert prefill.bs == decode.bs and prefill.cfg.num_hidden_layers == decode.cfg.num_hidden_layers
        self.prefill, self.decode = prefill, decode
        self.config = config or DisaggregationConfig(enable=True)
        self.stats = {"kv_bytes_transferred": 0, "handoffs": 0}

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams]) -> list[RequestOutput]:
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        chunk = self.config.prefill_chunk or len(prompts)
        if not self.decode.running:
            self.decode._ensure_out(max(p.max_tokens for p in plist))
        rids: list[str] = []
        results: dict[str, RequestOutput] = {}
        for lo in range(0, len(prompts), max(1, chunk)):
            hand = self.prefill.prefill_only(prompts[lo : lo + chunk], plist[lo : lo + chunk])
            for h, sp in zip(hand, plist[lo : lo + chunk]):
                self.stats["kv_bytes_transferred"] += h["kv"].numel() * h["kv"].element_size()
                self.stats["handoffs"] += 1
                rids.append(self.decode.add_prefilled(h, sp))
            # decode what is queued while the next chunk is prefilled (sequential here; two processes overlap the stages)
            for o in self.decode.step():
                results[o.request_id] = o
        while len(results) < len(rids):
            progressed = self.decode.step()
            for o in progressed:
                results[o.request_id] = o
            if not progressed and not self.decode.has_unfinished():
                break
        return [results[r] for r in rids]
