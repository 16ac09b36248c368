"""Architecture description of the decoder-only model families this framework trains and serves.

A ``ModelConfig`` can be built from a HuggingFace ``config.json`` (llama, qwen2, qwen3, qwen3_moe, mistral) so that
checkpoints and configs of the reference ecosystem load unchanged, and converts back with :meth:`to_hf_dict`.
The reference gets the same information from ``transformers.AutoConfig`` (``verl/utils/model.py:84-134``).
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional

__all__ = ["ModelConfig", "PRESETS"]


@dataclass
class ModelConfig:
    model_type: str = "qwen2"
    vocab_size: int = 152064
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    sliding_window: int = 0              # > 0: the checkpoint expects windowed attention; sequences up to the window are exact, longer ones are refused
    rope_scaling: Optional[dict] = None   # HF rope_scaling / rope_parameters mapping (linear, llama3, yarn); None or default: plain RoPE
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool = True          # qwen2: bias on q/k/v projections
    qk_norm: bool = False                # qwen3: RMSNorm on q and k heads
    mlp_act: str = "swiglu"              # "swiglu": gated SiLU MLP (gate/up fused); "xielu": up -> xIELU (learned per layer) -> down (Apertus)
    initializer_range: float = 0.02
    # mixture of experts (qwen3_moe)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    # heads
    value_head: bool = False             # scalar value head instead of lm_head (critic / reward model)
    vision: Optional[dict] = None        # vision-language models: fields of verl_b200.models.vision.VisionConfig
    pad_token_id: Optional[int] = 0
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        assert self.num_attention_heads % self.num_key_value_heads == 0

    # ------------------------------------------------------------------ derived sizes
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_parameters(self, include_embedding: bool = True) -> int:
        h, L = self.hidden_size, self.num_hidden_layers
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.attention_bias:
            attn += self.q_size + 2 * self.kv_size
        if self.qk_norm:
            attn += 2 * self.head_dim
        if self.is_moe:
            mlp = self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
        else:
            mlp = 3 * h * self.intermediate_size
        n = L * (attn + mlp + 2 * h) + h
        if include_embedding:
            n += self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return n

    # ------------------------------------------------------------------ HF interop
    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        def _text_rope_scaling(dd):
            rs = dd.get("rope_scaling") or dd.get("rope_parameters") or None
            if not rs:
                return None
            kind = rs.get("rope_type", rs.get("type", "default"))
            if kind in (None, "default", "mrope"):
                return None
            return {k: v for k, v in rs.items() if k != "rope_theta" and v is not None}

        mt = d.get("model_type", "llama")
        vision = None
        if mt in ("qwen2_vl", "qwen2_5_vl", "qwen3_vl"):
            # vision-language checkpoint: decoder fields sit in text_config (newer layout) or at the top level (older one)
            import dataclasses as _dc

            from verl_b200.models.vision import VisionConfig

            text = d.get("text_config") or {}
            vision = _dc.asdict(VisionConfig.from_hf_dict(d, text or None))
            vision["mrope_section"] = list(vision["mrope_section"])
            vision["fullatt_block_indexes"] = list(vision["fullatt_block_indexes"])
            vision["deepstack_visual_indexes"] = list(vision["deepstack_visual_indexes"])
            if mt == "qwen3_vl":      # Qwen3 decoder: per-head q/k norms, no projection biases
                d = {**{k: v for k, v in d.items() if k not in ("text_config", "vision_config")}, **text, "attention_bias": bool(text.get("attention_bias", False))}
                mt = "qwen3"
            else:
                d = {**{k: v for k, v in d.items() if k not in ("text_config", "vision_config")}, **text, "attention_bias": True}
                mt = "qwen2"
        known = dict(
            model_type=mt,
            vocab_size=d["vocab_size"],
            hidden_size=d["hidden_size"],
            intermediate_size=d.get("intermediate_size", 0),
            num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            head_dim=d.get("head_dim"),
            rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            rope_theta=d.get("rope_theta", (d.get("rope_parameters") or {}).get("rope_theta", 10000.0)),
            rope_scaling=_text_rope_scaling(d),
            sliding_window=int(d.get("sliding_window") or 0) if d.get("use_sliding_window", mt in ("mistral", "mixtral")) else 0,
            max_position_embeddings=d.get("max_position_embeddings", 32768),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
            attention_bias=d.get("attention_bias", mt == "qwen2"),
            qk_norm=mt in ("qwen3", "qwen3_moe", "apertus"),
            mlp_act="xielu" if mt == "apertus" else "swiglu",
            initializer_range=d.get("initializer_range", 0.02),
            num_experts=d.get("num_experts", d.get("num_local_experts", 0)) if "moe" in mt or "mixtral" in mt else 0,
            num_experts_per_tok=d.get("num_experts_per_tok", 0),
            moe_intermediate_size=d.get("moe_intermediate_size", 0),
            norm_topk_prob=d.get("norm_topk_prob", True),
            router_aux_loss_coef=d.get("router_aux_loss_coef", 0.0),
            pad_token_id=d.get("pad_token_id"),
            eos_token_id=d.get("eos_token_id") if not isinstance(d.get("eos_token_id"), list) else d["eos_token_id"][0],
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            vision=vision,
        )
        return cls(**known)

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls.from_hf_dict(json.loads(p.read_text()))

    def to_hf_dict(self) -> dict:
        arch = {"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
                "llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM"}.get(self.model_type, "LlamaForCausalLM")
        if self.value_head:
            arch = arch.replace("ForCausalLM", "ForTokenClassification")
        d = dict(
            architectures=[arch], model_type=self.model_type, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            intermediate_size=self.intermediate_size, num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads,
            head_dim=self.head_dim, rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta,
            max_position_embeddings=self.max_position_embeddings, tie_word_embeddings=self.tie_word_embeddings,
            attention_bias=self.attention_bias, initializer_range=self.initializer_range, hidden_act="xielu" if self.mlp_act == "xielu" else "silu",
            pad_token_id=self.pad_token_id, eos_token_id=self.eos_token_id, bos_token_id=self.bos_token_id,
            torch_dtype=self.torch_dtype,
        )
        if self.rope_scaling:
            d["rope_scaling"] = dict(self.rope_scaling)
        if self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob,
                     router_aux_loss_coef=self.router_aux_loss_coef)
        if self.value_head:
            d["num_labels"] = 1
        if self.vision:
            v = dict(self.vision)
            if v.get("variant") == "qwen3_vl":
                v.pop("variant")
                text = {k: d.pop(k) for k in list(d) if k not in ("architectures", "torch_dtype", "tie_word_embeddings")}
                text.update(model_type="qwen3_vl_text", rope_scaling={"rope_type": "default", "mrope_section": list(v.pop("mrope_section")),
                                                                      "mrope_interleaved": bool(v.pop("mrope_interleaved", True))})
                d.update(model_type="qwen3_vl", architectures=["Qwen3VLForConditionalGeneration"], image_token_id=v.pop("image_token_id"),
                         video_token_id=v.pop("video_token_id"), vision_start_token_id=v.pop("vision_start_token_id"), text_config=text)
                v["out_hidden_size"], v["hidden_size"] = v.pop("hidden_size"), v.pop("embed_dim")
                for k in ("mlp_ratio", "window_size", "fullatt_block_indexes", "tokens_per_second"):
                    v.pop(k, None)
                v["deepstack_visual_indexes"] = list(v["deepstack_visual_indexes"])
                d["vision_config"] = v
                return d
            for k in ("num_position_embeddings", "deepstack_visual_indexes", "mrope_interleaved"):
                v.pop(k, None)
            if v.get("variant", "qwen2_vl") != "qwen2_5_vl":
                v.pop("tokens_per_second", None)
            new = v.pop("variant", "qwen2_vl") == "qwen2_5_vl"
            d.update(model_type="qwen2_5_vl" if new else "qwen2_vl",
                     architectures=["Qwen2_5_VLForConditionalGeneration" if new else "Qwen2VLForConditionalGeneration"],
                     image_token_id=v.pop("image_token_id"), video_token_id=v.pop("video_token_id"), vision_start_token_id=v.pop("vision_start_token_id"),
                     rope_scaling={"type": "mrope", "mrope_section": list(v.pop("mrope_section"))})
            if new:       # the newer layout names the tower width hidden_size and the merger output out_hidden_size
                v["out_hidden_size"], v["hidden_size"] = v.pop("hidden_size"), v.pop("embed_dim")
                v.pop("mlp_ratio", None)
            else:
                for k in ("intermediate_size", "window_size", "fullatt_block_indexes"):
                    v.pop(k, None)
            d["vision_config"] = v
        return d

    def save_pretrained(self, path: str):
        Path(path).mkdir(parents=True, exist_ok=True)
        (Path(path) / "config.json").write_text(json.dumps(self.to_hf_dict(), indent=2))

    def replace(self, **kw) -> "ModelConfig":
        d = asdict(self)
        d.update(kw)
        return ModelConfig(**d)


PRESETS: dict[str, ModelConfig] = {
    # 2-layer plumbing model of the CPU/gloo correctness configuration
    "tiny-qwen2": ModelConfig(model_type="qwen2", vocab_size=2048, hidden_size=128, intermediate_size=512,
                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6,
                              rope_theta=1e4, tie_word_embeddings=True, max_position_embeddings=4096, torch_dtype="float32"),
    # vision-language plumbing model: 2-layer decoder + 2-block tower on 4×4 patches, image token ids inside the small vocabulary
    "tiny-qwen2-vl": ModelConfig(model_type="qwen2", vocab_size=2048, hidden_size=128, intermediate_size=512, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=True,
                                 max_position_embeddings=4096, torch_dtype="float32",
                                 vision=dict(depth=2, embed_dim=32, num_heads=2, mlp_ratio=2.0, in_channels=3, patch_size=4, temporal_patch_size=2,
                                             spatial_merge_size=2, hidden_size=128, image_token_id=2040, video_token_id=2041,
                                             vision_start_token_id=2042, mrope_section=[4, 6, 6])),
    # mixture-of-experts plumbing model (router replay, expert parallelism tests)
    "tiny-qwen3-moe": ModelConfig(model_type="qwen3_moe", vocab_size=2048, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, head_dim=16, qk_norm=True, rms_norm_eps=1e-6, rope_theta=1e4,
                                  num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, tie_word_embeddings=True,
                                  max_position_embeddings=4096, torch_dtype="float32"),
    "tiny-qwen2-gpu": ModelConfig(model_type="qwen2", vocab_size=4096, hidden_size=512, intermediate_size=1536,
                                  num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                                  rope_theta=1e4, max_position_embeddings=4096),
    "qwen2.5-0.5b": ModelConfig(model_type="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864,
                                num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2,
                                tie_word_embeddings=True),
    "qwen2.5-7b": ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                              num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6),
    "llama3.1-8b": ModelConfig(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                               num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, rope_theta=5e5,
                               attention_bias=False, rms_norm_eps=1e-5, max_position_embeddings=131072),
    "qwen3-8b": ModelConfig(model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                            num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                            attention_bias=False, qk_norm=True, rope_theta=1e6),
    "qwen3-30b-a3b": ModelConfig(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                                 num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                                 attention_bias=False, qk_norm=True, rope_theta=1e6, num_experts=128,
                                 num_experts_per_tok=8, moe_intermediate_size=768),
}
