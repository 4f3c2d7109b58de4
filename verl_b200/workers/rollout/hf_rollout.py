"""``generate()``-style rollout on the trainer's model: micro-batched, greedy / sampling / validation kwargs,
top-k / top-p, ``num_return_sequences`` and right-padding after EOS.

Parity target: ``verl/workers/rollout/hf_rollout.py:39-177`` (sampling-parameter precedence :56-92, output keys
``prompts/responses/input_ids/attention_mask/position_ids`` :130-170).
"""

from __future__ import annotations

import torch

from ...protocol import DataProto
from ...utils.tensordict_lite import TensorDict
from .naive.naive_rollout import NaiveRollout, filter_logits, last_token_logits

__all__ = ["HFRollout"]


class HFRollout(NaiveRollout):
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        bs = len(prompts)
        micro = int(self._cfg("micro_batch_size", bs) or bs)
        chunks = prompts.chunk(max(bs // micro, 1)) if bs >= micro and bs % max(bs // micro, 1) == 0 else [prompts]
        return DataProto.concat([self._generate_minibatch(c) for c in chunks])

    def _sampling_kwargs(self, prompts: DataProto) -> dict:
        mi = prompts.meta_info
        do_sample = mi.get("do_sample", self._cfg("do_sample", True))
        if not do_sample:
            return dict(do_sample=False, temperature=1.0, top_k=0, top_p=1.0, n=1)
        if mi.get("validate", False):
            vk = self._cfg("val_kwargs", {}) or {}
            g = vk.get if hasattr(vk, "get") else lambda k, d=None: getattr(vk, k, d)
            return dict(do_sample=True, temperature=g("temperature", 1.0), top_k=max(0, g("top_k", 0) or 0),
                        top_p=g("top_p", 1.0), n=1)
        return dict(do_sample=True, temperature=mi.get("temperature", self._cfg("temperature", 1.0)),
                    top_k=max(0, mi.get("top_k", self._cfg("top_k", 0)) or 0), top_p=mi.get("top_p", self._cfg("top_p", 1.0)),
                    n=int(mi.get("n", self._cfg("n", 1)) or 1))

    @torch.no_grad()
    def _generate_minibatch(self, prompts: DataProto) -> DataProto:
        kw = self._sampling_kwargs(prompts)
        idx, am = prompts.batch["input_ids"], prompts.batch["attention_mask"]
        pos = prompts.batch["position_ids"] if "position_ids" in prompts.batch.keys() else (torch.cumsum(am, -1) - 1).clamp_min(0)
        if kw["n"] > 1:
            idx, am, pos = (t.repeat_interleave(kw["n"], 0) for t in (idx, am, pos))
        eos = prompts.meta_info.get("eos_token_id", getattr(self.model_config, "eos_token_id", None))
        eos = [eos] if isinstance(eos, int) else list(eos or [])
        pad = prompts.meta_info.get("pad_token_id", getattr(self.model_config, "pad_token_id", 0)) or 0
        b, P = idx.shape
        R = int(self._cfg("response_length"))
        gen = None
        if prompts.meta_info.get("seed") is not None:
            gen = torch.Generator(device=idx.device).manual_seed(int(prompts.meta_info["seed"]))
        seq, mask, p = idx, am, pos
        done = torch.zeros(b, dtype=torch.bool, device=idx.device)
        for _ in range(R):
            logits = last_token_logits(self.module, seq, mask, p)
            if kw["do_sample"]:
                logits = filter_logits(logits / max(float(kw["temperature"]), 1e-8), int(kw["top_k"]), float(kw["top_p"]))
                nxt = torch.multinomial(torch.softmax(logits, -1), 1, generator=gen).squeeze(-1)
            else:
                nxt = logits.argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
            seq = torch.cat([seq, nxt[:, None]], 1)
            mask = torch.cat([mask, (~done).to(mask.dtype)[:, None]], 1)
            p = torch.cat([p, p[:, -1:] + (~done).to(p.dtype)[:, None]], 1)
            for e in eos:
                done = done | (nxt == e)
            if bool(done.all()):
                break
        short = P + R - seq.size(1)
        if short > 0:  # everyone stopped early: right-pad to the fixed response length
            seq = torch.cat([seq, seq.new_full((b, short), pad)], 1)
            mask = torch.cat([mask, mask.new_zeros(b, short)], 1)
            p = torch.cat([p, p[:, -1:].expand(b, short)], 1)
        batch = TensorDict({"prompts": seq[:, :P], "responses": seq[:, P:], "input_ids": seq, "attention_mask": mask,
                            "position_ids": p, "response_mask": mask[:, P:]}, batch_size=b)
        return DataProto(batch=batch, meta_info=dict(prompts.meta_info))
