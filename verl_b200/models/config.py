"""Architecture description of the decoder families the framework trains and serves.

One dataclass covers Llama / Mistral / Qwen2 / Qwen2.5 / Qwen3 dense models and Qwen3-MoE style sparse
models; it converts from and to HF ``config.json`` dictionaries so checkpoints stay interchangeable.
Reference: model families handled in ``verl/models/transformers/*`` and ``verl/utils/flops_counter.py``.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

__all__ = ["ModelConfig", "PRESETS", "get_preset", "NATIVE_FAMILIES"]

# architectures with a hand-scheduled decoder (own kernels, own backward, paged rollout engine); every other causal language
# model of the ``transformers`` library runs through ``models/generic.py``
NATIVE_FAMILIES = ("llama", "mistral", "qwen2", "qwen3", "qwen3_moe", "qwen2_moe", "mixtral", "phi3")


@dataclass
class ModelConfig:
    model_type: str = "qwen2"
    vocab_size: int = 512
    hidden_size: int = 128
    intermediate_size: int = 256
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None   # context extension of the rotary embedding: {rope_type: linear | llama3 | yarn, factor, ...}
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = False
    # mixture of experts (0 experts = dense MLP)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    shared_expert_intermediate_size: int = 0   # > 0: a dense expert every token passes through, scaled by a sigmoid gate
    router_aux_loss_coef: float = 0.0
    # tokens
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    initializer_range: float = 0.02
    extra: dict = field(default_factory=dict)
    # model-parallel shard description (a full model has both ends and local = global expert count)
    has_embedding: bool = True    # pipeline stage owns the token embedding
    has_head: bool = True         # pipeline stage owns the final norm and the LM/value head
    num_local_experts: int = 0    # expert-parallel shard: experts stored on this rank (0 = all)
    head_vocab_size: int = 0      # vocabulary-parallel shard: rows of the LM head stored on this rank (0 = all)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.model_type in ("qwen2", "qwen2_moe") and "attention_bias" not in self.extra.get("_explicit", ()):
            self.attention_bias = True
        if self.model_type in ("qwen3", "qwen3_moe"):
            self.qk_norm = True

    def local_shard(self, tp: int = 1, num_layers: Optional[int] = None, has_embedding: bool = True, has_head: bool = True,
                    ep: int = 1, vocab_parallel: bool = False) -> "ModelConfig":
        """Configuration of what ONE rank of a tensor x pipeline (x expert) parallel layout stores and computes: 1/tp of the
        attention heads and of the MLP width (column-parallel QKV / gate-up, row-parallel O / down), ``num_layers``
        consecutive layers, the embedding only on the first and the head only on the last stage, 1/ep of the experts."""
        import dataclasses

        assert self.num_attention_heads % tp == 0 and self.num_key_value_heads % tp == 0, "tp must divide the head counts"
        assert self.is_moe or self.intermediate_size % tp == 0
        # mixture-of-experts layers under tensor parallelism: every expert's (and the shared expert's) intermediate width is
        # cut over the tensor-parallel ranks (expert tensor parallelism = tp), the router stays replicated
        etp = tp if self.is_moe else 1
        assert not self.is_moe or (self.moe_intermediate_size % etp == 0 and self.shared_expert_intermediate_size % etp == 0), \
            "tp must divide the experts' intermediate sizes"
        c = dataclasses.replace(self, num_attention_heads=self.num_attention_heads // tp,
                                num_key_value_heads=self.num_key_value_heads // tp,
                                intermediate_size=self.intermediate_size // tp if not self.is_moe else self.intermediate_size,
                                moe_intermediate_size=self.moe_intermediate_size // etp,
                                shared_expert_intermediate_size=self.shared_expert_intermediate_size // etp,
                                num_hidden_layers=self.num_hidden_layers if num_layers is None else num_layers,
                                head_dim=self.head_dim, has_embedding=has_embedding, has_head=has_head,
                                num_local_experts=(self.num_experts // ep if self.is_moe and ep > 1 else 0),
                                head_vocab_size=(self.vocab_size // tp if vocab_parallel and tp > 1 and has_head
                                                 and not self.tie_word_embeddings and self.vocab_size % (8 * tp) == 0 else 0),
                                tie_word_embeddings=self.tie_word_embeddings and has_embedding and has_head, extra=dict(self.extra))
        return c

    # ------------------------------------------------------------------ derived sizes
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_generic(self) -> bool:
        """True for architectures that run as a library module under autograd (no hand-scheduled decoder)."""
        return bool(self.extra.get("generic"))

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    def num_parameters(self, value_head: bool = False) -> int:
        h, v = self.hidden_size, self.vocab_size
        per_layer = 2 * h + self.qkv_size * h + self.q_size * h
        if self.attention_bias:
            per_layer += self.qkv_size
        if self.qk_norm:
            per_layer += 2 * self.head_dim
        if self.is_moe:
            per_layer += self.num_experts * h + self.num_experts * 3 * h * self.moe_intermediate_size
            if self.shared_expert_intermediate_size:
                per_layer += 3 * h * self.shared_expert_intermediate_size + 8 * h
        else:
            per_layer += 3 * h * self.intermediate_size
        total = v * h + self.num_hidden_layers * per_layer + h
        if value_head:
            total += 8 * h
        elif not self.tie_word_embeddings:
            total += v * h
        return total

    @property
    def is_multimodal(self) -> bool:
        """True for vision-language architectures (a vision tower feeds placeholder tokens of the text stream)."""
        return self.is_generic and isinstance(self.extra.get("hf_config", {}).get("vision_config"), dict)

    # ------------------------------------------------------------------ HF interchange
    @classmethod
    def from_hf_dict(cls, d: dict[str, Any]) -> "ModelConfig":
        mt = d.get("model_type", "llama")
        if mt not in NATIVE_FAMILIES:
            return cls._generic_from_hf_dict(d)
        # rotary settings: older configurations keep ``rope_theta`` + ``rope_scaling`` at the top level, newer ones one
        # ``rope_parameters`` dict
        rp, rs = d.get("rope_parameters") or {}, d.get("rope_scaling") or {}
        theta = rp.get("rope_theta") or d.get("rope_theta") or 10000.0
        scaling = {**rs, **{k: v for k, v in rp.items() if k != "rope_theta"}}
        kind = scaling.get("rope_type") or scaling.get("type") or "default"
        scaling = dict(scaling, rope_type=kind) if kind != "default" else None
        window = d.get("sliding_window") if d.get("use_sliding_window", mt in ("mistral", "mixtral", "phi3")) else None
        windowed = window is not None and int(window) < int(d.get("max_position_embeddings", 32768))
        odd = (
            (d.get("partial_rotary_factor") or 1.0) != 1.0
            or str(d.get("hidden_act", "silu")) not in ("silu", "swish")
            or bool(d.get("mlp_bias", False))
            or (bool(d.get("attention_bias", False)) and mt not in ("qwen2", "qwen2_moe"))   # these families bias the output projection too
            or int(d.get("decoder_sparse_step", 1) or 1) != 1 or len(d.get("mlp_only_layers") or []) > 0  # dense layers among the sparse ones
        )
        if kind not in ("default", "linear", "llama3", "yarn") or windowed or odd:
            # rules the hand-scheduled decoder does not implement (sliding-window attention, other rotary variants): the
            # library module is exact for them
            return cls._generic_from_hf_dict(d)
        kw = dict(
            model_type=mt,
            vocab_size=d["vocab_size"],
            hidden_size=d["hidden_size"],
            intermediate_size=d.get("intermediate_size", 0),
            num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            head_dim=d.get("head_dim"),
            rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            rope_theta=float(theta), rope_scaling=scaling,
            max_position_embeddings=d.get("max_position_embeddings", 32768),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", mt in ("qwen2", "qwen2_moe"))),
            num_experts=d.get("num_experts", d.get("num_local_experts", 0)) or 0,
            num_experts_per_tok=d.get("num_experts_per_tok", 0) or 0,
            # Mixtral names its expert width ``intermediate_size``
            moe_intermediate_size=(d.get("moe_intermediate_size", 0) or 0) or (d.get("intermediate_size", 0) if mt == "mixtral" else 0),
            norm_topk_prob=bool(d.get("norm_topk_prob", mt != "qwen2_moe")),
            shared_expert_intermediate_size=(d.get("shared_expert_intermediate_size", 0) or 0) if mt == "qwen2_moe" else 0,
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id") if not isinstance(d.get("eos_token_id"), list) else d["eos_token_id"][0],
            pad_token_id=d.get("pad_token_id"),
            initializer_range=d.get("initializer_range", 0.02),
        )
        cfg = cls(**kw, extra={"_explicit": ("attention_bias",)})
        return cfg

    @classmethod
    def _generic_from_hf_dict(cls, d: dict[str, Any]) -> "ModelConfig":
        """Description of an architecture outside ``NATIVE_FAMILIES``: the sizes the framework reports and plans with
        (FLOPs estimate, token ids) are read leniently; the complete library configuration travels in ``extra``."""
        t = d.get("text_config") if isinstance(d.get("text_config"), dict) else d
        heads = t.get("num_attention_heads", 1)
        eos = d.get("eos_token_id", t.get("eos_token_id"))
        # latent attention (DeepSeek-V2/V3): the score width is nope + rope dims
        head_dim = t.get("head_dim") or ((t.get("qk_nope_head_dim", 0) + t.get("qk_rope_head_dim", 0)) or None)
        return cls(model_type=d.get("model_type"), vocab_size=t.get("vocab_size", d.get("vocab_size", 0)),
                   hidden_size=t.get("hidden_size", 0), intermediate_size=t.get("intermediate_size", 0) or 0,
                   num_hidden_layers=t.get("num_hidden_layers", 0), num_attention_heads=heads,
                   num_key_value_heads=t.get("num_key_value_heads", heads) or heads, head_dim=head_dim,
                   rms_norm_eps=t.get("rms_norm_eps", 1e-6), max_position_embeddings=t.get("max_position_embeddings", 32768),
                   tie_word_embeddings=bool(d.get("tie_word_embeddings", t.get("tie_word_embeddings", False))),
                   bos_token_id=d.get("bos_token_id", t.get("bos_token_id")), eos_token_id=eos[0] if isinstance(eos, list) else eos,
                   pad_token_id=d.get("pad_token_id", t.get("pad_token_id")), initializer_range=t.get("initializer_range", 0.02),
                   extra={"generic": True, "hf_config": dict(d), "_explicit": ("attention_bias",)})

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def to_hf_dict(self) -> dict[str, Any]:
        if self.is_generic:
            return dict(self.extra["hf_config"])
        arch = {
            "qwen2": "Qwen2ForCausalLM",
            "qwen3": "Qwen3ForCausalLM",
            "qwen3_moe": "Qwen3MoeForCausalLM",
            "qwen2_moe": "Qwen2MoeForCausalLM",
            "llama": "LlamaForCausalLM",
            "mistral": "MistralForCausalLM",
            "mixtral": "MixtralForCausalLM",
            "phi3": "Phi3ForCausalLM",
        }.get(self.model_type, "LlamaForCausalLM")
        d = {
            "architectures": [arch],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            **({"rope_scaling": dict(self.rope_scaling)} if self.rope_scaling else {}),
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "hidden_act": "silu",
            "torch_dtype": "bfloat16",
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_id,
            "pad_token_id": self.pad_token_id,
            "initializer_range": self.initializer_range,
        }
        if self.is_moe and self.model_type == "mixtral":
            d.update(num_local_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     intermediate_size=self.moe_intermediate_size)
        elif self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob)
            if self.shared_expert_intermediate_size:
                d.update(shared_expert_intermediate_size=self.shared_expert_intermediate_size, decoder_sparse_step=1, mlp_only_layers=[])
        return d

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_hf_dict(), f, indent=2)

    def to_dict(self) -> dict:
        return asdict(self)


PRESETS: dict[str, ModelConfig] = {
    # BASELINE config 1 (CPU/gloo oracle)
    "tiny-qwen2": ModelConfig(model_type="qwen2", vocab_size=512, hidden_size=128, intermediate_size=256,
                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4,
                              eos_token_id=2, pad_token_id=0),
    "qwen2.5-0.5b": ModelConfig(model_type="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864,
                                num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2,
                                rope_theta=1e6, tie_word_embeddings=True, eos_token_id=151645, pad_token_id=151643),
    "qwen2.5-7b": ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                              num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6,
                              eos_token_id=151645, pad_token_id=151643),
    "llama-3.1-8b": ModelConfig(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                                num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                                rope_theta=5e5, rms_norm_eps=1e-5, eos_token_id=128001, pad_token_id=128001,
                                max_position_embeddings=131072,
                                rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                              "original_max_position_embeddings": 8192}),
    "qwen3-30b-a3b": ModelConfig(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                                 num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                                 rope_theta=1e6, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                                 eos_token_id=151645, pad_token_id=151643),
    "tiny-moe": ModelConfig(model_type="qwen3_moe", vocab_size=512, hidden_size=128, intermediate_size=256,
                            num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                            num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, eos_token_id=2,
                            pad_token_id=0),
    "tiny-qwen2-moe": ModelConfig(model_type="qwen2_moe", vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, num_experts=8, num_experts_per_tok=2,
                                  moe_intermediate_size=64, shared_expert_intermediate_size=128, norm_topk_prob=False,
                                  eos_token_id=2, pad_token_id=0),
    "tiny-qwen3": ModelConfig(model_type="qwen3", vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                              num_attention_heads=4, num_key_value_heads=2, head_dim=32, eos_token_id=2, pad_token_id=0),
    "tiny-llama": ModelConfig(model_type="llama", vocab_size=512, hidden_size=128, intermediate_size=256,
                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, eos_token_id=2,
                              pad_token_id=0),
}


def get_preset(name: str) -> ModelConfig:
    import copy

    key = name.lower().replace("_", "-")
    for k, v in PRESETS.items():
        if k == key or key.endswith(k) or k in key:
            return copy.deepcopy(v)
    raise KeyError(f"unknown model preset '{name}' (known: {sorted(PRESETS)})")
