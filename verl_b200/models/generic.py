"""Model families without a hand-scheduled decoder: any causal language model of the ``transformers`` library
(DeepSeek-V2/V3 with latent attention, GPT-OSS, Gemma, GLM, OLMo, ...) trained through the same engine.

The hand-written decoder (``models/decoder.py``) covers the Llama / Qwen / Mistral / Mixtral / Phi-3 families with its own
kernels and its own backward. Every other architecture runs here as a library module under autograd, but keeps the
engine's memory plan: all parameters of the module are re-pointed at views of ONE flat working buffer
(:class:`ModuleFlatParams`), gradients are accumulated into the flat fp32 main-gradient buffer as soon as autograd has
produced them, so the sharded optimizer, the gradient reduce-scatter, checkpoints and weight sync are the engine's usual
code. The LM head goes through the fused log-prob / entropy kernel (no [tokens, vocabulary] logits) unless the
architecture alters its logits (soft-capping, head bias). The engine's packed token stream is handed to the module as
right-padded rows with a 2-D mask (the one format all families treat alike) and gathered back to the stream afterwards.

This path trades speed for breadth: it is the counterpart of the reference's generic module engine
(``verl/workers/engine/fsdp/transformer_impl.py:230-380`` builds any ``AutoModelForCausalLM`` /
``AutoModelForTokenClassification``; packed inputs with position ids :560-640).
"""

from __future__ import annotations

import math
from typing import Iterator, Optional

import torch

from .config import ModelConfig
from .weights import ALIGN, ParamSpec

__all__ = ["ModuleFlatParams", "GenericCausalLM", "GenericRolloutEngine", "build_hf_module"]


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


def build_hf_module(cfg: ModelConfig, dtype: torch.dtype, seed: int = 0, value_head: bool = False,
                    attn_implementation: Optional[str] = None) -> torch.nn.Module:
    """Random-initialised library module for the architecture stored in ``cfg.extra['hf_config']``."""
    from transformers import AutoConfig, AutoModelForCausalLM, AutoModelForImageTextToText

    d = dict(cfg.extra["hf_config"])
    mt = d.pop("model_type")
    d.pop("architectures", None)
    d.pop("torch_dtype", None)
    d.pop("dtype", None)
    hf_cfg = AutoConfig.for_model(mt, **d)
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(seed)
        # without an explicit choice the library picks its best supported attention (fused SDPA where the family has it)
        # ("native" names this framework's own attention kernels, which serve the hand-scheduled families only)
        kw = {"attn_implementation": attn_implementation} if attn_implementation and attn_implementation != "native" else {}
        auto = AutoModelForImageTextToText if cfg.is_multimodal else AutoModelForCausalLM
        module = auto.from_config(hf_cfg, dtype=dtype, **kw)
        if value_head:
            h = hf_cfg.get_text_config().hidden_size
            module.v_head = torch.nn.Linear(h, 1, bias=False, dtype=dtype)
            torch.nn.init.normal_(module.v_head.weight, std=cfg.initializer_range)
    return module


class ModuleFlatParams:
    """The parameters of a ``torch.nn.Module`` stored in one flat buffer, with the interface of
    :class:`verl_b200.models.weights.FlatParams` (``flat``, ``views``, ``offsets``, ``main_grad``, HF-named views)."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", value_head: bool = False, pad_to: int = 1,
                 buffer: Optional[torch.Tensor] = None, seed: int = 0, module: Optional[torch.nn.Module] = None,
                 attn_implementation: Optional[str] = None):
        self.cfg, self.dtype, self.value_head = cfg, dtype, value_head
        self._seed = seed
        self._attn_implementation = attn_implementation
        self.module = module if module is not None else build_hf_module(cfg, dtype, seed, value_head, attn_implementation)
        self.module.to(device)  # buffers (rotary tables, routing biases) move; parameters are re-pointed below
        named = list(self.module.named_parameters())  # tied parameters appear once
        self.specs = [ParamSpec(n, tuple(p.shape), "module", p.dim() >= 2, self._layer_of(n)) for n, p in named]
        self.offsets: dict[str, int] = {}
        off = 0
        for s in self.specs:
            self.offsets[s.name] = off
            off += _round_up(s.numel, ALIGN)
        self.numel = self.dense_numel = _round_up(off, ALIGN * max(1, pad_to))
        self.flat = buffer if buffer is not None else torch.zeros(self.numel, dtype=dtype, device=device)
        assert self.flat.numel() == self.numel
        self.main_grad: Optional[torch.Tensor] = None
        self.views: dict[str, torch.Tensor] = {}
        self._grad_views: dict[str, torch.Tensor] = {}
        for (n, p), s in zip(named, self.specs):
            o = self.offsets[n]
            v = self.flat[o : o + s.numel].view(*s.shape)
            if buffer is None:
                v.copy_(p.data)      # a buffer handed in is authoritative (merged checkpoints, shared storage)
            p.data = v
            self.views[n] = v
            p.register_post_accumulate_grad_hook(self._make_hook(n))

    @staticmethod
    def _layer_of(name: str) -> int:
        parts = name.split(".")
        for a, b in zip(parts, parts[1:]):
            if a == "layers" and b.isdigit():
                return int(b)
        return -1

    def _make_hook(self, name: str):
        def hook(p: torch.Tensor) -> None:
            # autograd's gradient (working precision) is folded into the fp32 main-gradient buffer and dropped at once,
            # so no second full-size gradient copy lives through the backward
            g = self._grad_views.get(name)
            if g is None:
                raise RuntimeError("backward without a gradient buffer: call optimizer_zero_grad() before the step")
            g.add_(p.grad)
            p.grad = None

        return hook

    # ------------------------------------------------------------------ gradients
    def attach_main_grad(self, grad_buffer: Optional[torch.Tensor] = None) -> None:
        self.main_grad = grad_buffer if grad_buffer is not None else torch.zeros(self.numel, dtype=torch.float32,
                                                                                 device=self.flat.device)
        for s in self.specs:
            o = self.offsets[s.name]
            self._grad_views[s.name] = self.main_grad[o : o + s.numel].view(*s.shape)

    def detach_main_grad(self) -> None:
        self.main_grad = None
        self._grad_views.clear()

    def zero_grad(self) -> None:
        if self.main_grad is not None:
            self.main_grad.zero_()

    # ------------------------------------------------------------------ access
    def __getitem__(self, name: str) -> torch.Tensor:
        return self.views[name]

    def decay_mask_ranges(self) -> list[tuple[int, int, bool]]:
        return [(self.offsets[s.name], self.offsets[s.name] + _round_up(s.numel, ALIGN), s.decay) for s in self.specs]

    def layer_range(self, i: int) -> tuple[int, int]:
        names = [s for s in self.specs if s.layer == i]
        last = names[-1]
        return self.offsets[names[0].name], self.offsets[last.name] + _round_up(last.numel, ALIGN)

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.module.get_output_embeddings().weight

    def init_weights(self, seed: int = 0, std: Optional[float] = None) -> None:
        """The module was initialised by the library's own rules at construction; another seed re-draws it."""
        if seed == self._seed:
            return
        fresh = build_hf_module(self.cfg, self.dtype, seed, self.value_head, self._attn_implementation)
        for n, p in fresh.named_parameters():
            self.views[n].copy_(p.data)
        self._seed = seed

    # ------------------------------------------------------------------ HF interchange
    def hf_views(self, prefix: str = "") -> Iterator[tuple[str, torch.Tensor]]:
        """Checkpoint-named tensors: the module's own parameter names are the library's checkpoint names."""
        for s in self.specs:
            yield prefix + s.name, self.views[s.name]

    def hf_state_dict(self, clone: bool = False) -> dict[str, torch.Tensor]:
        return {k: (v.clone() if clone else v) for k, v in self.hf_views()}

    def load_hf_state_dict(self, sd: dict[str, torch.Tensor], strict: bool = True) -> list[str]:
        missing = []
        for name, view in self.hf_views():
            if name in sd:
                view.copy_(sd[name].to(view.dtype))
            else:
                missing.append(name)
        if strict and missing:
            raise KeyError(f"missing tensors: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
        return missing

    def copy_from(self, other) -> None:
        self.flat.copy_(other.flat.to(self.flat.dtype))

    def named_parameters(self) -> Iterator[tuple[str, torch.Tensor]]:
        return iter(self.views.items())


def _logprob_entropy_from_logits(logits: torch.Tensor, labels: torch.Tensor):
    logp = torch.log_softmax(logits.float(), -1)
    lp = logp.gather(-1, labels.long()[:, None]).squeeze(-1)
    ent = -(logp.exp() * logp).sum(-1)
    return lp, ent


class GenericCausalLM:
    """A library module behind the interface the engines use (``forward_logprobs`` / ``forward_values`` /
    ``forward_logits`` on packed batches). Differentiable outputs are ordinary autograd tensors."""

    def __init__(self, cfg: ModelConfig, params: ModuleFlatParams, recompute: str = "auto"):
        self.cfg, self.params = cfg, params
        self.module = params.module
        # vision-language models: the trunk is the module that merges the vision tower's output into the text stream
        self.multimodal = bool(cfg.is_multimodal)
        self.trunk = self.module.model if self.multimodal or not hasattr(self.module, "get_decoder") else self.module.get_decoder()
        hf = self.module.config.get_text_config()
        self.softcap = float(getattr(hf, "final_logit_softcapping", 0.0) or 0.0)
        head = self.module.get_output_embeddings()
        self._plain_head = self.softcap == 0.0 and getattr(head, "bias", None) is None
        self.recompute = recompute
        if recompute != "none" and getattr(self.module, "supports_gradient_checkpointing", False):
            self.module.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
        self.module.eval()
        # attributes the engines set on the hand-written decoder; none of them applies here
        self.sp = self.tp = self.ep = self.tsp = self.router_replay = self.offloader = self.vocab_parallel = None
        self.mlp_tile_tokens = 0
        self.keep_layers_fn = None
        self.stats_hook = None

    def activation_bytes_per_layer(self, num_tokens: int) -> int:
        return 0  # recomputation is all-or-nothing here (the library's gradient checkpointing)

    # ------------------------------------------------------------------ forward
    def _hidden(self, batch, need_grad: bool, mm_inputs: Optional[dict] = None) -> torch.Tensor:
        assert getattr(batch, "expand_index", None) is None, "shared-prefix packing needs the hand-written decoder"
        # gradient checkpointing and dropout follow the module's training flag
        self.module.train(bool(need_grad) and self.recompute != "none")
        # The packed stream is laid out as right-padded rows with a 2-D mask: the one input format every family of the
        # library handles exactly (families differ in whether they derive packed-sequence masks from position ids, and
        # sliding-window / hybrid layers build their own masks from the 2-D one).
        dev = batch.input_ids.device
        lens = (batch.cu_seqlens_cpu[1:] - batch.cu_seqlens_cpu[:-1]).to(torch.int64)
        b, width = lens.numel(), int(lens.max())
        row = torch.repeat_interleave(torch.arange(b), lens).to(dev)
        col = (torch.arange(int(lens.sum())) - torch.repeat_interleave(batch.cu_seqlens_cpu[:-1].to(torch.int64), lens)).to(dev)
        ids = torch.zeros(b, width, dtype=torch.int64, device=dev).index_put_((row, col), batch.input_ids.long())
        pos = torch.zeros(b, width, dtype=torch.int64, device=dev).index_put_((row, col), batch.positions.long())
        mask = torch.zeros(b, width, dtype=torch.int64, device=dev).index_put_((row, col), torch.ones_like(row))
        if self.multimodal:
            # multi-axis rotary positions (time / height / width of the image patches) follow from the placeholder tokens and
            # the grids: the library derives them from the mask; ``mm_inputs`` holds the processor's tensors of this
            # micro-batch's rows, concatenated in row order (pixel_values, image_grid_thw, ...)
            out = self.trunk(input_ids=ids, attention_mask=mask, use_cache=False, **(mm_inputs or {}))
        else:
            assert not mm_inputs, "multi-modal inputs for a text-only architecture"
            out = self.trunk(input_ids=ids, attention_mask=mask, position_ids=pos, use_cache=False)
        return out.last_hidden_state[row, col]

    def _head(self, hS: torch.Tensor, labels: torch.Tensor, temperature: float):
        if self._plain_head:
            from ..utils.kernel.linear_cross_entropy import linear_cross_entropy

            return linear_cross_entropy(hS, self.params.lm_head_weight, labels, temperature)
        logits = self.module.get_output_embeddings()(hS).float()
        if self.softcap:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        return _logprob_entropy_from_logits(logits / temperature, labels)

    def forward_logprobs(self, batch, labels: torch.Tensor, temperature: float = 1.0, need_grad: Optional[bool] = None,
                         positions: Optional[torch.Tensor] = None, stage_input=None,
                         position_labels: Optional[torch.Tensor] = None, mm_inputs: Optional[dict] = None):
        """(log_probs, entropy) per packed position (fp32), or per entry of ``positions``."""
        need_grad = torch.is_grad_enabled() if need_grad is None else need_grad
        with torch.set_grad_enabled(bool(need_grad)):
            h = self._hidden(batch, need_grad, mm_inputs)
            if positions is not None:
                h = h.index_select(0, positions)
                labels = position_labels if position_labels is not None else labels.index_select(0, positions)
            lp, ent = self._head(h, labels, temperature)
        return lp.float(), ent.float()

    def forward_values(self, batch, need_grad: Optional[bool] = None, stage_input=None, mm_inputs: Optional[dict] = None) -> torch.Tensor:
        need_grad = torch.is_grad_enabled() if need_grad is None else need_grad
        with torch.set_grad_enabled(bool(need_grad)):
            h = self._hidden(batch, need_grad, mm_inputs)
            return self.module.v_head(h)[:, 0].float()

    @torch.no_grad()
    def forward_hidden(self, batch) -> torch.Tensor:
        return self._hidden(batch, False)

    @torch.no_grad()
    def forward_logits(self, batch, mm_inputs: Optional[dict] = None) -> torch.Tensor:
        logits = self.module.get_output_embeddings()(self._hidden(batch, False, mm_inputs)).float()
        if self.softcap:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        return logits


class GenericRolloutEngine:
    """Batched sampling with the library module and its key/value cache, behind the part of the rollout engine's
    interface the workers use (``generate`` returning ``RequestOutput``s with the sampled tokens' log-probs). It reads
    the trainer's flat parameter buffer in place, so there is no weight sync. Prompts are served in chunks of
    ``max_num_seqs`` left-padded rows; a chunk ends when all of its rows have stopped."""

    def __init__(self, cfg: ModelConfig, params: ModuleFlatParams, *, max_num_seqs: int = 64, eos_token_id=None, seed: int = 0,
                 **unused):
        self.cfg, self.params = cfg, params
        self.module = params.module
        self.max_num_seqs = max(1, int(max_num_seqs))
        eos = eos_token_id if eos_token_id is not None else cfg.eos_token_id
        self.eos = set([eos] if isinstance(eos, int) else list(eos or []))
        self.seed = int(seed)
        self._calls = 0
        self.stats = {"generated_tokens": 0, "prefill_tokens": 0, "steps": 0}

    def resume_kv_cache(self) -> None:
        return None

    def release_kv_cache(self) -> None:
        return None

    def clear_kv_cache(self) -> None:
        return None  # the cache of a generate() call dies with the call

    @torch.no_grad()
    def generate(self, prompts, params, mm_inputs=None):
        """``mm_inputs``: per prompt, the processor's tensors of its images / videos (or None); the prompt ids already hold
        the placeholder tokens."""
        from ..workers.rollout.native.engine import RequestOutput
        from ..workers.rollout.naive.naive_rollout import filter_logits

        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        outs: list = [None] * len(prompts)
        dev = self.params.flat.device
        was_training = self.module.training
        self.module.eval()
        for c0 in range(0, len(prompts), self.max_num_seqs):
            rows = list(range(c0, min(len(prompts), c0 + self.max_num_seqs)))
            b, P = len(rows), max(len(prompts[i]) for i in rows)
            ids = torch.zeros(b, P, dtype=torch.int64)
            mask = torch.zeros(b, P, dtype=torch.int64)
            for r, i in enumerate(rows):
                n = len(prompts[i])
                ids[r, P - n :] = torch.tensor(list(prompts[i]), dtype=torch.int64)
                mask[r, P - n :] = 1
            ids, mask = ids.to(dev), mask.to(dev)
            sp = [plist[i] for i in rows]
            temp = torch.tensor([max(float(s.temperature), 0.0) for s in sp], dtype=torch.float32, device=dev)
            greedy = temp <= 0
            max_new = max(int(s.max_tokens) for s in sp)
            gens = []
            for r, s in enumerate(sp):
                g = torch.Generator(device="cpu")
                g.manual_seed(int(s.seed) if s.seed is not None else (self.seed * 1000003 + self._calls * 7919 + rows[r]))
                gens.append(g)
            toks: list[list[int]] = [[] for _ in rows]
            lps: list[list[float]] = [[] for _ in rows]
            reason = ["length"] * b
            done = torch.zeros(b, dtype=torch.bool)
            pos = (mask.cumsum(-1) - 1).clamp_min(0)
            cache, step_ids, step_pos = None, ids, pos
            self.stats["prefill_tokens"] += int(mask.sum())
            multimodal = bool(self.cfg.is_multimodal)
            first_kw = {}
            if mm_inputs is not None and multimodal:
                per_key: dict = {}
                for i in rows:
                    for k, v in (mm_inputs[i] or {}).items():
                        if isinstance(v, torch.Tensor):
                            per_key.setdefault(k, []).append(v)
                first_kw = {k: torch.cat(v, 0).to(dev) for k, v in per_key.items()}
            for t in range(max_new):
                if multimodal:
                    # multi-axis rotary positions: the library derives them from the mask and the grids at the prefill and
                    # continues them from its stored offsets on the cached steps
                    out = self.module(input_ids=step_ids, attention_mask=mask, past_key_values=cache, use_cache=True,
                                      **(first_kw if t == 0 else {}))
                else:
                    out = self.module(input_ids=step_ids, attention_mask=mask, position_ids=step_pos, past_key_values=cache,
                                      use_cache=True)
                cache = out.past_key_values
                logits = out.logits[:, -1].float()
                scaled = logits / torch.where(greedy, torch.ones_like(temp), temp)[:, None]
                logp = torch.log_softmax(scaled, -1).cpu()
                nxt = torch.empty(b, dtype=torch.int64)
                for r, s in enumerate(sp):
                    if done[r]:
                        nxt[r] = 0
                        continue
                    if greedy[r]:
                        nxt[r] = int(logp[r].argmax())
                    else:
                        f = filter_logits(logp[r : r + 1].clone(), int(s.top_k) if s.top_k and s.top_k > 0 else 0, float(s.top_p))
                        nxt[r] = int(torch.multinomial(torch.softmax(f, -1), 1, generator=gens[r]))
                    toks[r].append(int(nxt[r]))
                    lps[r].append(float(logp[r, nxt[r]]))
                    stop = (not s.ignore_eos and int(nxt[r]) in self.eos) or int(nxt[r]) in set(s.stop_token_ids or ())
                    if stop:
                        done[r], reason[r] = True, "completed"
                    elif len(toks[r]) >= int(s.max_tokens):
                        done[r] = True
                self.stats["steps"] += 1
                if bool(done.all()):
                    break
                step_ids = nxt.to(dev)[:, None]
                mask = torch.cat([mask, torch.ones(b, 1, dtype=mask.dtype, device=dev)], 1)
                step_pos = step_pos[:, -1:] + 1
            for r, i in enumerate(rows):
                self.stats["generated_tokens"] += len(toks[r])
                outs[i] = RequestOutput(request_id=f"g{self._calls}-{i}", prompt_ids=list(prompts[i]), token_ids=toks[r],
                                        log_probs=lps[r] if sp[r].logprobs else None, stop_reason=reason[r])
        self._calls += 1
        self.module.train(was_training)
        return outs
