"""Model families beyond the default decoder: parity with the Hugging Face implementations."""

import pytest
import torch



def test_apertus_family_matches_hf():
    """Apertus: un-gated MLP with the xIELU activation (two learned curvature scalars per layer), per-head q/k norms, its own
    norm names — logits equal Hugging Face, and names / config round-trip."""
    try:
        from transformers import ApertusConfig, ApertusForCausalLM
    except ImportError:
        pytest.skip("this transformers build has no Apertus")
    from verl_b200.models.config import ModelConfig
    from verl_b200.models.transformer import DecoderLM, PackedBatch

    torch.manual_seed(0)
    hf_cfg = ApertusConfig(vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                           max_position_embeddings=256, rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, tie_word_embeddings=False,
                           hidden_act="xielu", dtype="float32")
    hf = ApertusForCausalLM(hf_cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "alpha_" in n or "norm" in n:
                p.add_(0.2 * torch.randn_like(p))
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict()).replace(torch_dtype="float32", rms_norm_eps=hf_cfg.rms_norm_eps)
    assert cfg.mlp_act == "xielu" and cfg.qk_norm and not cfg.attention_bias
    ours = DecoderLM(cfg, dtype=torch.float32)
    ours.load_hf_state_dict({k: v for k, v in hf.state_dict().items() if not k.endswith((".beta", ".eps"))})
    ids = torch.randint(0, 320, (23,))
    with torch.no_grad():
        want = hf(input_ids=ids[None]).logits[0]
        got = ours(PackedBatch(ids, torch.arange(23, dtype=torch.int32), torch.tensor([0, 23], dtype=torch.int32)), return_logits=True)["logits"]
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()
    exported = dict(ours.hf_named_tensors())
    sd = hf.state_dict()
    for k, v in exported.items():
        assert torch.equal(v.reshape(sd[k].shape), sd[k]), k
    assert "model.layers.1.mlp.act_fn.alpha_n" in exported and "model.layers.0.feedforward_layernorm.weight" in exported
    assert ModelConfig.from_hf_dict(cfg.to_hf_dict() | {"model_type": "apertus"}).mlp_act == "xielu"
    # a freshly initialised model starts from the published activation parameters
    fresh = DecoderLM(cfg, dtype=torch.float32, seed=1)
    assert abs(float(torch.nn.functional.softplus(fresh.layers[0].mlp.act_alpha_p)) - 0.8) < 1e-6


def test_apertus_generates_in_the_rollout_engine_and_trains_in_the_engine():
    """The family goes through the paged rollout engine (greedy tokens equal repeated full forwards) and the sharded-DP engine
    (a step runs, the activation's learned scalars receive gradients); tensor-parallel / fp8 rollouts of it are refused."""
    from tests.test_engine_on_cpu import loss_fn, make_batch
    from verl_b200.models.config import PRESETS
    from verl_b200.models.transformer import DecoderLM, PackedBatch
    from verl_b200.workers.engine.fsdp.engine import FSDPEngine
    from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams

    cfg = PRESETS["tiny-qwen2"].replace(model_type="apertus", mlp_act="xielu", qk_norm=True, attention_bias=False, tie_word_embeddings=False)
    model = DecoderLM(cfg, dtype=torch.float32, seed=5).eval()
    prompt = [11, 12, 13, 14, 15]
    out = InferenceEngine(model, max_num_seqs=4, max_model_len=64, num_blocks=16, enforce_eager=True).generate(
        [prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))[0]
    ids = list(prompt)
    for _ in range(5):
        t = torch.tensor(ids)
        with torch.no_grad():
            lg = model(PackedBatch(t, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32)), return_logits=True)["logits"]
        ids.append(int(lg[-1].argmax()))
    assert list(out.token_ids) == ids[-5:]
    with pytest.raises(NotImplementedError, match="un-gated MLP"):
        InferenceEngine(model, max_num_seqs=4, max_model_len=64, num_blocks=16, quantization="fp8")
    eng = FSDPEngine(cfg, {"seed": 1}, {"lr": 1e-3, "clip_grad": 1.0}, {})
    eng.initialize()
    data = make_batch()
    data.meta_info["micro_batch_size_per_gpu"] = 4
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(data, loss_fn)
    assert eng.model.layers[0].mlp.act_alpha_p.main_grad.abs().sum() > 0 and eng.model.layers[1].mlp.up_proj.main_grad.abs().sum() > 0
    assert eng.optimizer_step() > 0


@pytest.mark.parametrize("scaling", [
    {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    {"rope_type": "linear", "factor": 4.0},
    {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64, "beta_fast": 32, "beta_slow": 1},
])
def test_rope_scaling_types_match_hf(scaling):
    """Llama-3.1-style, linear and YaRN rotary scaling: logits of a sequence longer than the original context equal Hugging Face,
    the rollout engine decodes with the same tables, and the mapping survives the config round trip."""
    from transformers import LlamaConfig, LlamaForCausalLM

    from verl_b200.models.config import ModelConfig
    from verl_b200.models.transformer import DecoderLM, PackedBatch
    from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams

    torch.manual_seed(0)
    hf_cfg = LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=256, rope_parameters={"rope_theta": 10000.0, **scaling}, tie_word_embeddings=False)
    hf = LlamaForCausalLM(hf_cfg).float().eval()
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict()).replace(torch_dtype="float32", rms_norm_eps=hf_cfg.rms_norm_eps)
    assert cfg.rope_scaling["rope_type"] == scaling["rope_type"] and "rope_theta" not in cfg.rope_scaling
    ours = DecoderLM(cfg, dtype=torch.float32)
    ours.load_hf_state_dict(hf.state_dict())
    ids = torch.randint(0, 320, (150,))
    with torch.no_grad():
        want = hf(input_ids=ids[None]).logits[0]
        got = ours(PackedBatch(ids, torch.arange(150, dtype=torch.int32), torch.tensor([0, 150], dtype=torch.int32)), return_logits=True)["logits"]
    assert torch.allclose(got, want, atol=3e-4, rtol=1e-3), (got - want).abs().max()
    plain = DecoderLM(cfg.replace(rope_scaling=None), dtype=torch.float32)
    plain.load_hf_state_dict(hf.state_dict())
    with torch.no_grad():
        off = plain(PackedBatch(ids, torch.arange(150, dtype=torch.int32), torch.tensor([0, 150], dtype=torch.int32)), return_logits=True)["logits"]
    assert (off - want).abs().max() > 1e-3                                   # the scaling matters for this input
    out = InferenceEngine(ours.eval(), max_num_seqs=2, max_model_len=192, num_blocks=8, enforce_eager=True).generate(
        [ids[:100].tolist()], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))[0]
    seq = ids[:100].tolist()
    for _ in range(3):
        t = torch.tensor(seq)
        with torch.no_grad():
            lg = ours(PackedBatch(t, torch.arange(len(seq), dtype=torch.int32), torch.tensor([0, len(seq)], dtype=torch.int32)), return_logits=True)["logits"]
        seq.append(int(lg[-1].argmax()))
    assert list(out.token_ids) == seq[-3:]
    assert ModelConfig.from_hf_dict(cfg.to_hf_dict()).rope_scaling == cfg.rope_scaling


def test_sliding_window_checkpoints_are_exact_up_to_the_window_and_refused_beyond():
    from verl_b200.models.config import ModelConfig
    from verl_b200.models.transformer import DecoderLM, PackedBatch
    from verl_b200.workers.rollout.engine import InferenceEngine

    d = dict(model_type="mistral", vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
             max_position_embeddings=256, sliding_window=32, rope_theta=10000.0, torch_dtype="float32")
    cfg = ModelConfig.from_hf_dict(d)
    assert cfg.sliding_window == 32 and ModelConfig.from_hf_dict({**d, "model_type": "qwen2", "use_sliding_window": False}).sliding_window == 0
    m = DecoderLM(cfg, dtype=torch.float32)
    ok = torch.randint(0, 320, (32,))
    m(PackedBatch(ok, torch.arange(32, dtype=torch.int32), torch.tensor([0, 32], dtype=torch.int32)), return_logits=True)
    long = torch.randint(0, 320, (40,))
    with pytest.raises(NotImplementedError, match="sliding-window"):
        m(PackedBatch(long, torch.arange(40, dtype=torch.int32), torch.tensor([0, 40], dtype=torch.int32)), return_logits=True)
    with pytest.raises(NotImplementedError, match="sliding-window"):
        InferenceEngine(m, max_num_seqs=2, max_model_len=64, num_blocks=8)
    InferenceEngine(m, max_num_seqs=2, max_model_len=32, num_blocks=8)
