"""The in-house decoder must reproduce HuggingFace transformers' Qwen2 / Llama / Qwen3 forward given the same weights."""

import pytest
import torch

from verl_b200.models.config import ModelConfig
from verl_b200.models.transformer import DecoderLM, PackedBatch, hf_to_native_state_dict


def _hf_model(cfg: ModelConfig):
    import transformers

    d = cfg.to_hf_dict()
    d.pop("architectures")
    cls = {"qwen2": (transformers.Qwen2Config, transformers.Qwen2ForCausalLM), "llama": (transformers.LlamaConfig, transformers.LlamaForCausalLM),
           "qwen3": (transformers.Qwen3Config, transformers.Qwen3ForCausalLM)}[cfg.model_type]
    d.pop("model_type")
    d.pop("torch_dtype", None)
    hf_cfg = cls[0](**d, attn_implementation="eager")
    torch.manual_seed(0)
    return cls[1](hf_cfg).float().eval()


@pytest.mark.parametrize("mt,bias,qk", [("qwen2", True, False), ("llama", False, False), ("qwen3", False, True)])
def test_logits_match_transformers(mt, bias, qk):
    cfg = ModelConfig(model_type=mt, vocab_size=512, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, rope_theta=1e4, attention_bias=bias, qk_norm=qk, tie_word_embeddings=False,
                      max_position_embeddings=256, torch_dtype="float32")
    hf = _hf_model(cfg)
    with torch.no_grad():
        for p in hf.parameters():          # make biases / norms non-trivial
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    mine = DecoderLM(cfg, dtype=torch.float32)
    mine.load_hf_state_dict(hf.state_dict())
    lens = [7, 12, 3]
    ids = [torch.randint(0, 512, (n,)) for n in lens]
    packed = torch.cat(ids)
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    cu = torch.tensor([0, 7, 19, 22], dtype=torch.int32)
    with torch.no_grad():
        out = mine(PackedBatch(packed, pos, cu), return_logits=True)["logits"]
        ref = torch.cat([hf(input_ids=x[None]).logits[0] for x in ids])
    assert torch.allclose(out, ref, atol=2e-4, rtol=1e-4), (out - ref).abs().max()


def test_hf_name_roundtrip():
    cfg = ModelConfig(model_type="qwen2", vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, tie_word_embeddings=True, torch_dtype="float32")
    m = DecoderLM(cfg, dtype=torch.float32)
    sd = {k: v.clone() for k, v in m.hf_named_tensors()}
    assert "model.layers.1.self_attn.k_proj.bias" in sd and "lm_head.weight" not in sd
    native = hf_to_native_state_dict(cfg, sd)
    for k, v in m.named_parameters():
        assert torch.equal(native[k], v)


def test_logprob_entropy_head_matches_logits_path():
    cfg = ModelConfig(model_type="qwen2", vocab_size=300, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, torch_dtype="float32")
    m = DecoderLM(cfg, dtype=torch.float32)
    ids = torch.randint(0, 300, (10,))
    pb = PackedBatch(ids, torch.arange(10, dtype=torch.int32), torch.tensor([0, 10], dtype=torch.int32))
    labels = torch.roll(ids, -1)
    out = m(pb, labels=labels, temperature=0.7, return_logits=True)
    logits = out["logits"] / 0.7
    ref_lp = torch.log_softmax(logits, -1).gather(-1, labels[:, None]).squeeze(-1)
    p = torch.softmax(logits, -1)
    ref_ent = -(p * torch.log(p)).sum(-1)
    assert torch.allclose(out["log_probs"], ref_lp, atol=1e-5) and torch.allclose(out["entropy"], ref_ent, atol=1e-5)
