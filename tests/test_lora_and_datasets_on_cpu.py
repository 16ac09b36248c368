"""LoRA adapters through the engine, and the supervised datasets."""

import torch

from tests.test_engine_on_cpu import loss_fn, make_batch
from verl_b200.models.config import PRESETS
from verl_b200.models.lora import apply_lora, lora_state_dict, merge_lora_, merged_hf_named_tensors
from verl_b200.models.transformer import DecoderLM, PackedBatch
from verl_b200.utils.config import Config
from verl_b200.utils.dataset.samplers import DifficultyCurriculumSampler
from verl_b200.utils.dataset.sft_dataset import MultiTurnSFTDataset, RMDataset
from verl_b200.utils.tokenizer import ByteChatTokenizer
from verl_b200.workers.engine.fsdp.engine import FSDPEngine


def _logits(m, ids):
    pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
    with torch.no_grad():
        return m(pb, return_logits=True)["logits"]


def test_lora_is_identity_at_init_trains_only_adapters_and_merges():
    base = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=1)
    ids = torch.arange(10, 30)
    want = _logits(base, ids)
    apply_lora(base, rank=4, alpha=8, target_modules=["q_proj", "down_proj"])
    assert torch.allclose(_logits(base, ids), want, atol=1e-6)          # B starts at zero
    assert set(base.lora_config["targets"]) == {"qkv_proj", "down_proj"} and len(lora_state_dict(base)) == 2 * 2 * 2
    eng = FSDPEngine(Config({"preset": "tiny-qwen2", "lora_rank": 4, "lora_alpha": 8}), {"seed": 1}, {"lr": 1e-2, "weight_decay": 0.0}, {})
    eng.initialize()
    n_train = sum(p.numel() for p in eng.store.params)
    assert n_train < 0.1 * sum(p.numel() for p in eng.model.parameters()) and all("lora_" in n for n in eng.store.names)
    frozen_before = eng.model.layers[0].mlp.down_proj.clone()
    for _ in range(2):
        eng.train_batch(make_batch(), loss_fn)
    assert torch.equal(eng.model.layers[0].mlp.down_proj, frozen_before)
    assert eng.model.layers[0].mlp.lora_B_down_proj.abs().sum() > 0
    got = _logits(eng.model, ids)
    exported = dict(eng.get_per_tensor_param()[0])
    fresh = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=1)
    fresh.load_hf_state_dict(exported)
    assert torch.allclose(_logits(fresh, ids), got, atol=1e-4)
    merge_lora_(eng.model)
    assert torch.allclose(_logits(eng.model, ids), got, atol=1e-4) and not lora_state_dict(eng.model)
    assert len(dict(merged_hf_named_tensors(eng.model))) == len(exported)


def test_merge_lora_script_exports_merged_weights_and_a_peft_adapter(tmp_path):
    """A LoRA run's checkpoint holds the adapters only; the merge tool folds them into the base weights and also writes them in
    the PEFT layout (fused projections split per HF module)."""
    import json

    from safetensors.torch import load_file

    from verl_b200.models.hf_io import save_hf_weights
    from verl_b200.scripts.merge_lora import merge_lora_checkpoint

    base = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=1)
    base_dir = tmp_path / "base"
    base_dir.mkdir()
    PRESETS["tiny-qwen2"].save_pretrained(str(base_dir))
    save_hf_weights(base.hf_named_tensors(), str(base_dir))
    eng = FSDPEngine(Config({"path": str(base_dir), "lora_rank": 4, "lora_alpha": 8}), {"seed": 1, "model_dtype": "float32"},
                     {"lr": 1e-2, "weight_decay": 0.0}, {})
    eng.initialize()
    for _ in range(2):
        eng.train_batch(make_batch(), loss_fn)
    ids = torch.arange(10, 30)
    want = _logits(eng.model, ids)
    eng.save_checkpoint(str(tmp_path / "ckpt"), global_step=2)
    meta = json.load(open(tmp_path / "ckpt" / "fsdp_config.json"))
    assert meta["lora"]["rank"] == 4 and "qkv_proj" in meta["lora"]["targets"]
    info = merge_lora_checkpoint(str(base_dir), str(tmp_path / "ckpt"), str(tmp_path / "merged"), dtype=torch.float32)
    merged = {}
    for fn in (tmp_path / "merged").iterdir():
        if fn.suffix == ".safetensors":
            merged.update(load_file(str(fn)))
    fresh = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=9)
    fresh.load_hf_state_dict(merged)
    assert torch.allclose(_logits(fresh, ids), want, atol=2e-2)          # merged weights are stored in bf16
    ad = load_file(str(tmp_path / "merged" / "lora_adapter" / "adapter_model.safetensors"))
    acfg = json.load(open(tmp_path / "merged" / "lora_adapter" / "adapter_config.json"))
    assert acfg["r"] == 4 and {"q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "o_proj", "down_proj"} == set(acfg["target_modules"])
    cfg = PRESETS["tiny-qwen2"]
    kq = "base_model.model.model.layers.0.self_attn.q_proj"
    assert ad[kq + ".lora_A.weight"].shape == (4, cfg.hidden_size) and ad[kq + ".lora_B.weight"].shape == (cfg.num_attention_heads * cfg.head_dim, 4)
    kv = "base_model.model.model.layers.0.self_attn.v_proj.lora_B.weight"
    full_b = eng.model.layers[0].self_attn.lora_B_qkv_proj.detach()
    assert torch.allclose(ad[kv].float(), full_b[-cfg.num_key_value_heads * cfg.head_dim:].float(), atol=1e-2)
    assert info["num_adapter_tensors"] == len(ad)


def test_multiturn_sft_dataset_masks_only_assistant_tokens():
    tok = ByteChatTokenizer()
    rows = [{"messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
                          {"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "4"}], "tools": None}]
    ds = MultiTurnSFTDataset(rows=rows, tokenizer=tok, max_length=160)
    item = ds[0]
    n = int(item["attention_mask"].sum())
    ids, lm = item["input_ids"][:n], item["loss_mask"][:n]
    targets = ids[1:][lm[:-1].bool()]
    assert tok.decode(targets.tolist()) == "yo<|im_end|>\n4<|im_end|>\n"
    assert item["position_ids"][n - 1] == n - 1 and lm[n - 1] == 0
    rm = RMDataset(rows=[{"prompt": "q: ", "chosen": "good", "rejected": "bad"}], tokenizer=tok, max_length=16)[0]
    assert rm["input_ids"].shape == (2, 16) and rm["attention_mask"][0].sum() == len("q: good") + 1


def test_curriculum_sampler_prefers_medium_difficulty():
    from verl_b200.protocol import DataProto

    s = DifficultyCurriculumSampler(list(range(6)), explore=0.0)
    batch = DataProto.from_dict(tensors={"token_level_scores": torch.tensor([[1.0], [0.0], [0.5], [1.0], [0.0], [0.45]])},
                                non_tensors={"index": [0, 1, 2, 3, 4, 5]})
    s.update(batch)
    order = list(iter(s))
    assert order[0] == 2 and order[1] == 5 and sorted(order) == list(range(6))


def test_rollout_serves_the_trained_adapters(tmp_path):
    """A LoRA policy is generated from as it is trained: the rollout engine applies the live adapters on top of the shared base
    weights (no merged copy, no weight hand-off), so after updates the sampler's log-probs still equal the trainer's recomputation;
    fp8 / tensor-parallel replicas cannot apply adapters unmerged and are refused at the engine (the worker gives them a merged copy)."""
    import pytest

    from tests.test_trainer_e2e_on_cpu import OV
    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.utils.config import load_config
    from verl_b200.workers.rollout.engine import InferenceEngine

    cfg = load_config("ppo_trainer", OV + [f"trainer.default_local_dir={tmp_path}/ckpt", "actor_rollout_ref.model.lora_rank=4", "actor_rollout_ref.model.lora_alpha=8",
                                           "actor_rollout_ref.actor.optim.lr=5e-2", "trainer.total_training_steps=3"])
    tr = PPOTrainer(cfg, reward_fn=load_reward_manager(cfg, None), val_reward_fn=None)
    tr.init_workers()
    w = tr.actor_rollout_wg.worker
    assert not w._rollout_owns_model and w.rollout.model is w.actor.engine.model and w.actor.engine.model.lora_config["rank"] == 4
    it = iter(tr.train_dataloader)
    for step in (1, 2, 3):
        tr.global_steps = step
        m = tr.step(next(it))
        assert m["training/rollout_probs_diff_max"] < 1e-5, (step, m["training/rollout_probs_diff_max"])
    assert w.actor.engine.model.layers[0].self_attn.lora_B_qkv_proj.abs().sum() > 0            # the adapters did move
    assert w.checkpoint_manager.last_stats["path"] == "resident_shared"
    with pytest.raises(NotImplementedError, match="unmerged"):
        InferenceEngine(w.actor.engine.model, max_num_seqs=4, max_model_len=64, num_blocks=16, quantization="fp8")
