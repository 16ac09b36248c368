"""Vision-language family against the Hugging Face Qwen2-VL implementation (tiny random model, fp32, CPU): vision tower
output, 3-stream rope index and the logits of a sequence that holds an image."""

import pytest
import torch

from verl_b200.models.config import ModelConfig
from verl_b200.models.transformer import PackedBatch
from verl_b200.models.vision import VisionConfig, VisionLanguageModel, get_rope_index, mrope_tables

transformers = pytest.importorskip("transformers")


def _hf_model():
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    torch.manual_seed(0)
    cfg = Qwen2VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, rope_theta=10000.0, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]},
                         tie_word_embeddings=False),
        vision_config=dict(depth=2, embed_dim=32, num_heads=2, mlp_ratio=2, in_channels=3, patch_size=4, temporal_patch_size=2,
                           spatial_merge_size=2, hidden_size=64),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503)
    return Qwen2VLForConditionalGeneration(cfg).float().eval()


def _ours(hf):
    cfg = ModelConfig(model_type="qwen2", vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, rope_theta=10000.0, max_position_embeddings=512, attention_bias=True, rms_norm_eps=1e-5, torch_dtype="float32")
    vcfg = VisionConfig(depth=2, embed_dim=32, num_heads=2, mlp_ratio=2.0, patch_size=4, temporal_patch_size=2, spatial_merge_size=2, hidden_size=64,
                        image_token_id=500, video_token_id=501, vision_start_token_id=502, mrope_section=(2, 3, 3))
    m = VisionLanguageModel(cfg, vcfg, dtype=torch.float32, device=torch.device("cpu"))
    m.load_hf_state_dict(hf.state_dict())
    return m.eval()


def _sample():
    g = torch.Generator().manual_seed(1)
    grid = torch.tensor([[1, 4, 6], [1, 2, 2]])                   # two images: 24 and 4 patches → 6 and 1 merged tokens
    pixels = torch.randn(int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 4 * 4, generator=g)
    text = lambda n: torch.randint(1, 400, (n,), generator=g).tolist()
    ids = text(5) + [502] + [500] * 6 + [503] + text(4) + [502] + [500] * 1 + [503] + text(7)
    return torch.tensor(ids), pixels, grid


def test_vision_tower_matches_hf():
    hf = _hf_model()
    ours = _ours(hf)
    _, pixels, grid = _sample()
    with torch.no_grad():
        want = hf.model.visual(pixels, grid_thw=grid)
        want = want.pooler_output if hasattr(want, "pooler_output") else want
        got = ours.visual(pixels, grid)
    if isinstance(want, (tuple, list)):
        want = torch.cat(list(want), 0)
    assert got.shape == want.shape == (7, 64)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), (got - want).abs().max()


def test_rope_index_and_logits_match_hf():
    hf = _hf_model()
    ours = _ours(hf)
    ids, pixels, grid = _sample()
    pos3, delta = get_rope_index(ids, grid, ours.vcfg)
    import inspect

    kw = {"mm_token_type_ids": (ids == 500).long()[None]} if "mm_token_type_ids" in inspect.signature(hf.model.get_rope_index).parameters else {}
    want_pos, want_delta = hf.model.get_rope_index(ids[None], image_grid_thw=grid, attention_mask=torch.ones_like(ids)[None], **kw)[:2]
    assert torch.equal(pos3, want_pos[:, 0]) and delta == int(want_delta.reshape(-1)[0])
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=torch.ones_like(ids)[None],
                  position_ids=want_pos).logits[0]
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        got = ours(pb, pixel_values=pixels, image_grid_thw=grid, mrope_positions=pos3, return_logits=True)["logits"]
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()
    # padded layout: masked positions are skipped and get position 0
    mask = torch.cat([torch.zeros(3, dtype=torch.long), torch.ones_like(ids)])
    padded = torch.cat([torch.zeros(3, dtype=torch.long), ids])
    p2, d2 = get_rope_index(padded, grid, ours.vcfg, attention_mask=mask)
    assert torch.equal(p2[:, 3:], pos3) and d2 == delta and int(p2[:, :3].abs().sum()) == 0


def test_mrope_tables_reduce_to_plain_rope_for_text():
    pos = torch.arange(11)
    cos, sin = mrope_tables(pos[None].expand(3, -1), 16, 10000.0, (2, 3, 3))
    inv = 1.0 / (10000.0 ** (torch.arange(0, 16, 2).float() / 16))
    assert torch.allclose(cos, (pos[:, None].float() * inv).cos()) and torch.allclose(sin, (pos[:, None].float() * inv).sin())


def _vl_config():
    return ModelConfig(model_type="qwen2", vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, rope_theta=10000.0, max_position_embeddings=512, attention_bias=True, torch_dtype="float32",
                       vision=dict(depth=2, embed_dim=32, num_heads=2, mlp_ratio=2.0, in_channels=3, patch_size=4, temporal_patch_size=2,
                                   spatial_merge_size=2, hidden_size=64, image_token_id=500, video_token_id=501, vision_start_token_id=502,
                                   mrope_section=[2, 3, 3]))


def _vl3_config():
    """The same plumbing size in the Qwen3-VL family: Qwen3 decoder, interleaved rotary streams, deep-stack features after layers 0 and 1."""
    return ModelConfig(model_type="qwen3", vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, rope_theta=10000.0, max_position_embeddings=512, attention_bias=False, qk_norm=True,
                       torch_dtype="float32",
                       vision=dict(depth=2, embed_dim=32, num_heads=2, in_channels=3, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
                                   hidden_size=64, image_token_id=500, video_token_id=501, vision_start_token_id=502, mrope_section=[4, 2, 2],
                                   variant="qwen3_vl", intermediate_size=48, num_position_embeddings=36, deepstack_visual_indexes=[0, 1],
                                   mrope_interleaved=True))


def test_config_round_trips_through_the_hf_layout(tmp_path):
    cfg = _vl_config()
    cfg.save_pretrained(str(tmp_path))
    back = ModelConfig.from_pretrained(str(tmp_path))
    assert {k: back.vision[k] for k in cfg.vision} == cfg.vision and back.hidden_size == 64 and back.model_type == "qwen2"
    import json

    d = json.loads((tmp_path / "config.json").read_text())
    assert d["model_type"] == "qwen2_vl" and d["vision_config"]["embed_dim"] == 32 and d["rope_scaling"]["mrope_section"] == [2, 3, 3]
    # the nested text_config layout of newer checkpoints parses to the same thing
    text_keys = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "rope_theta",
                 "max_position_embeddings", "rms_norm_eps", "rope_scaling", "head_dim")
    nested = {k: v for k, v in d.items() if k not in text_keys}
    nested["text_config"] = {k: d[k] for k in text_keys}
    assert ModelConfig.from_hf_dict(nested).vision == back.vision


@pytest.mark.parametrize("family", ["qwen2_vl", "qwen3_vl"])
def test_engine_trains_a_vision_language_model_on_image_prompts(tmp_path, family):
    """The sharded-DP engine with a vision-language config: log-probs of a batch whose prompts hold images equal a direct
    forward of the model per sequence, the vision tower receives gradients, and an optimizer step changes it."""
    import numpy as np

    from verl_b200.protocol import DataProto
    from verl_b200.workers.engine.fsdp.engine import FSDPEngine

    v3 = family == "qwen3_vl"
    eng = FSDPEngine(_vl3_config() if v3 else _vl_config(), {"seed": 3, "model_dtype": "float32"}, {"lr": 1e-3, "clip_grad": 1.0}, {})
    eng.initialize()
    assert type(eng.model).__name__ == "VisionLanguageModel"
    g = torch.Generator().manual_seed(5)
    P, R, bs = 16, 6, 3
    rows, mm = [], []
    for i, grid in enumerate([[[1, 4, 4]], [], [[1, 2, 2], [1, 2, 4]]]):
        ids = []
        for t, h, w in grid:
            ids += [502] + [500] * (t * h * w // 4) + [503]
        ids += torch.randint(1, 400, (4,), generator=g).tolist()
        rows.append(ids)
        n_patch = sum(t * h * w for t, h, w in grid)
        mm.append({"pixel_values": torch.randn(n_patch, 96, generator=g), "image_grid_thw": torch.tensor(grid).reshape(-1, 3)} if grid else {})
    input_ids = torch.zeros(bs, P + R, dtype=torch.long)
    att = torch.zeros(bs, P + R, dtype=torch.long)
    for i, ids in enumerate(rows):
        resp = torch.randint(1, 400, (R - i,), generator=g).tolist()
        input_ids[i, P - len(ids):P] = torch.tensor(ids)
        att[i, P - len(ids):P] = 1
        input_ids[i, P:P + len(resp)] = torch.tensor(resp)
        att[i, P:P + len(resp)] = 1
    pos = torch.clip(torch.cumsum(att, -1) - 1, min=0)
    data = DataProto.from_dict(tensors={"input_ids": input_ids, "attention_mask": att, "position_ids": pos, "responses": input_ids[:, P:],
                                        "response_mask": att[:, P:], "advantages": torch.randn(bs, R, generator=g),
                                        "old_log_probs": torch.zeros(bs, R), "ref_log_prob": torch.zeros(bs, R)},
                               non_tensors={"multi_modal_inputs": np.array(mm, dtype=object)},
                               meta_info={"micro_batch_size_per_gpu": 2, "temperature": 1.0})
    lp = eng.infer_batch(data)["model_output"]["log_probs"]
    from verl_b200.models.vision import VisionConfig

    v = dict(eng.cfg.vision)
    vcfg = VisionConfig(**{**v, "mrope_section": tuple(v["mrope_section"])})
    for i in range(bs):
        ids = input_ids[i][att[i].bool()]
        grid = mm[i].get("image_grid_thw")
        pos3, _ = get_rope_index(ids, grid, vcfg)
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        with torch.no_grad():
            logits = eng.model(pb, pixel_values=mm[i].get("pixel_values"), image_grid_thw=grid, mrope_positions=pos3, return_logits=True)["logits"]
        ref = torch.log_softmax(logits.float(), -1)
        n_prompt = int(att[i, :P].sum())
        for t in range(int(att[i, P:].sum())):
            assert abs(lp[i, t] - ref[n_prompt - 1 + t, ids[n_prompt + t]]) < 1e-4
    from tests.test_engine_on_cpu import loss_fn

    last = eng.model.visual.merger.linear_fc2.weight if v3 else eng.model.visual.merger.mlp[2].weight
    before = last.detach().clone()
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(data, loss_fn)
    assert eng.model.visual.patch_embed.proj.weight.main_grad.abs().sum() > 0
    if v3:      # the deep-stack merger and the position table are trained through the decoder's stream (the features added after the LAST
        # decoder layer only change the image rows themselves, which carry no loss: only the first merger of this 2-layer model learns)
        assert eng.model.visual.deepstack_merger_list[0].linear_fc1.weight.main_grad.abs().sum() > 0
        assert eng.model.visual.deepstack_merger_list[1].linear_fc1.weight.main_grad.abs().sum() == 0
        assert eng.model.visual.pos_embed.weight.main_grad.abs().sum() > 0
    gn = eng.optimizer_step()
    assert gn > 0 and not torch.equal(before, last)
    exported = dict(eng.get_per_tensor_param()[0])
    assert ("model.visual.patch_embed.proj.weight" if v3 else "visual.patch_embed.proj.weight") in exported and "model.layers.0.self_attn.q_proj.weight" in exported
    # checkpoint → merger → the same tensors under Hugging Face names, and a config that parses back as vision-language
    from verl_b200.model_merger.base_model_merger import ModelMergerConfig
    from verl_b200.model_merger.fsdp_model_merger import FSDPModelMerger

    ckpt = str(tmp_path / "ckpt")
    eng.save_checkpoint(ckpt, global_step=1)
    assert {k: v for k, v in ModelConfig.from_pretrained(ckpt + "/huggingface").vision.items() if k in eng.cfg.vision} == eng.cfg.vision
    sd = FSDPModelMerger(ModelMergerConfig(operation="merge", backend="fsdp", local_dir=ckpt, target_dir=str(tmp_path / "hf"),
                                           hf_model_config_path=ckpt + "/huggingface"))._merge()
    assert sd.keys() == exported.keys()
    for k in exported:
        assert sd[k].shape == exported[k].shape and torch.allclose(sd[k].float(), exported[k].float(), atol=1e-2, rtol=1e-2), k


def test_image_patches_match_the_hf_processor():
    import numpy as np
    from PIL import Image

    from verl_b200.utils.dataset.vision_utils import expand_image_tokens, image_to_patches, process_image, smart_resize

    assert smart_resize(100, 200) == (112, 196) and smart_resize(10, 10) == (56, 56)
    h, w = smart_resize(4000, 3000)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 14 * 14 * 4 * 1280
    rng = np.random.default_rng(0)
    img = Image.fromarray(rng.integers(0, 255, (90, 150, 3), dtype=np.uint8))
    small = process_image({"image": img})
    assert (small.height, small.width) == smart_resize(90, 150)
    pix, grid = image_to_patches(small)
    assert pix.shape == (grid[0, 1] * grid[0, 2], 3 * 2 * 14 * 14)
    try:
        from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor

        proc = Qwen2VLImageProcessor()
        want = proc(images=[small], do_resize=False, return_tensors="pt")
    except Exception as e:  # noqa: BLE001 - the processor class moved or needs a backend that is not installed
        pytest.skip(f"Hugging Face image processor unavailable: {e}")
    assert torch.equal(want["image_grid_thw"], grid)
    assert torch.allclose(want["pixel_values"].float(), pix, atol=1e-5)
    assert expand_image_tokens([1, 500, 2, 500], torch.tensor([[1, 4, 4], [1, 2, 6]]), 500) == [1] + [500] * 4 + [2] + [500] * 3


def test_dataset_builds_multimodal_rows(tmp_path):
    import io

    import numpy as np
    import pandas as pd
    from PIL import Image

    from verl_b200.utils.dataset.rl_dataset import RLHFDataset, collate_fn

    class Tok:
        pad_token_id, chat_template = 0, None

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [500 if w == "<image>" else 501 if w == "<video>" else 1 + (hash(w) % 300) for w in text.split()]}

    buf = io.BytesIO()
    Image.fromarray(np.random.default_rng(1).integers(0, 255, (60, 60, 3), dtype=np.uint8)).save(buf, format="PNG")
    df = pd.DataFrame({"prompt": [[{"role": "user", "content": "look <image> and tell"}], [{"role": "user", "content": "no picture here"}]],
                       "images": [[{"bytes": buf.getvalue()}], []], "data_source": ["geo3k", "geo3k"]})
    f = tmp_path / "d.parquet"
    df.to_parquet(f)
    vision = dict(patch_size=4, temporal_patch_size=2, spatial_merge_size=2, image_token_id=500, mrope_section=[2, 3, 3])
    ds = RLHFDataset(str(f), Tok(), {"max_prompt_length": 96, "vision": vision, "image_min_pixels": 256, "image_max_pixels": 1024})
    a, b = ds[0], ds[1]
    g = a["multi_modal_inputs"]["image_grid_thw"]
    n_img_tok = int(g[0, 1] * g[0, 2]) // 4
    assert int((a["input_ids"] == 500).sum()) == n_img_tok and a["multi_modal_inputs"]["pixel_values"].shape == (int(g[0, 1] * g[0, 2]), 96)
    assert a["position_ids"].shape == (4, 96) and b["position_ids"].shape == (4, 96) and b["multi_modal_inputs"] == {}
    live = a["attention_mask"].bool()
    assert int(a["position_ids"][2][live].max()) < int(a["position_ids"][0][live].max())      # the image block advances less than its token count
    assert torch.equal(b["position_ids"][0], b["position_ids"][1])                            # text only: all streams equal
    batch = collate_fn([a, b])
    assert batch["position_ids"].shape == (2, 4, 96) and len(batch["multi_modal_inputs"]) == 2
    # a row with a video (six frames as arrays) before an image: grids and patches follow the order of the marks in the prompt
    frames = [np.random.default_rng(2).integers(0, 255, (32, 32, 3), dtype=np.uint8) for _ in range(6)]
    ds.df = pd.DataFrame({"prompt": [[{"role": "user", "content": "watch <video> then look <image> and compare"}]],
                          "images": [[{"bytes": buf.getvalue()}]], "videos": [[{"frames": frames, "fps": 2.0}]], "data_source": ["v"]})
    ds.vision = dict(vision, video_token_id=501, tokens_per_second=2)
    c = ds[0]
    gv = c["multi_modal_inputs"]["image_grid_thw"]
    assert gv.shape == (2, 3) and int(gv[0, 0]) == 3 and int(gv[1, 0]) == 1                          # 6 frames = 3 temporal patches, then the image
    assert int((c["input_ids"] == 501).sum()) == int(gv[0].prod()) // 4 and int((c["input_ids"] == 500).sum()) == int(gv[1].prod()) // 4
    assert c["multi_modal_inputs"]["pixel_values"].shape[0] == int(gv[0].prod() + gv[1].prod())
    assert c["multi_modal_inputs"]["grid_t_scale"].tolist() == [2.0, 1.0]                           # 2 frames per patch at 2 fps = 1 s, x 2 tokens per second
    live = c["attention_mask"].bool()
    vid = (c["input_ids"] == 501) & live
    assert sorted(set((c["position_ids"][1][vid] - c["position_ids"][1][vid].min()).tolist())) == [0, 2, 4]   # temporal stream advances by 2 per patch


@pytest.mark.parametrize("family", ["qwen2_vl", "qwen3_vl"])
def test_rollout_generates_from_image_prompts_like_a_full_forward(family):
    """Greedy decoding with images through the paged rollout engine equals greedy decoding by repeated full forwards of the
    model (per-token rotary tables at prefill, position offset after the image grid at decode; for Qwen3-VL also the deep-stack
    features added after the first layers at prefill); identical token ids with different images are not shared as one prefix."""
    from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams

    torch.manual_seed(0)
    model = VisionLanguageModel(_vl_config() if family == "qwen2_vl" else _vl3_config(), dtype=torch.float32, device=torch.device("cpu"), seed=11).eval()
    if family == "qwen3_vl":
        with torch.no_grad():      # the seeded init leaves deep-stack outputs tiny: scale them up so that dropping them would change tokens
            for mod in model.visual.deepstack_merger_list:
                mod.linear_fc2.weight.mul_(40.0)
    g = torch.Generator().manual_seed(2)
    grid = torch.tensor([[1, 4, 4]])
    prompt = [7, 8, 502] + [500] * 4 + [503, 9, 10, 11]
    mm_a = {"pixel_values": torch.randn(16, 96, generator=g), "image_grid_thw": grid}
    mm_b = {"pixel_values": torch.randn(16, 96, generator=g), "image_grid_thw": grid}
    text = [5, 6, 7, 8, 9]
    eng = InferenceEngine(model, max_num_seqs=8, max_model_len=64, num_blocks=32, enforce_eager=True)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = eng.generate([prompt, prompt, text, prompt], sp, multi_modal=[mm_a, mm_b, None, mm_a])

    def greedy(ids, mm, n):
        ids = list(ids)
        for _ in range(n):
            t = torch.tensor(ids)
            pos3, _ = get_rope_index(t, mm["image_grid_thw"] if mm else None, model.vcfg)
            pb = PackedBatch(t, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
            with torch.no_grad():
                logits = model(pb, pixel_values=mm["pixel_values"] if mm else None, image_grid_thw=mm["image_grid_thw"] if mm else None,
                               mrope_positions=pos3, return_logits=True)["logits"]
            ids.append(int(logits[-1].argmax()))
        return ids[-n:]

    assert list(outs[0].token_ids) == greedy(prompt, mm_a, 6)
    assert list(outs[1].token_ids) == greedy(prompt, mm_b, 6)
    assert list(outs[2].token_ids) == greedy(text, None, 6)
    assert list(outs[3].token_ids) == list(outs[0].token_ids)
    assert list(outs[0].token_ids) != list(outs[1].token_ids) or not torch.equal(mm_a["pixel_values"], mm_b["pixel_values"])


@pytest.mark.parametrize("mode", ["sync", "async"])
def test_grpo_step_on_image_prompts_end_to_end(tmp_path, mode):
    """GRPO through the trainer with a vision-language actor: parquet prompts with images → rollout with the tower at
    prefill → old/ref log-probs and the update on multimodal micro-batches. On-policy, so the first PPO KL is ~0 — which
    only holds if rollout and trainer agree on image embeddings and rotary positions."""
    import io

    import numpy as np
    import pandas as pd
    from PIL import Image

    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.utils.config import load_config

    rng = np.random.default_rng(3)
    rows = []
    for i in range(8):
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 255, (16 + 8 * (i % 2), 24, 3), dtype=np.uint8)).save(buf, format="PNG")
        rows.append({"prompt": [{"role": "user", "content": f"<image> what is {i} plus {i}?"}], "images": [{"bytes": buf.getvalue()}],
                     "data_source": "synthetic/mod7", "reward_model": {"ground_truth": str(i % 7)}})
    f = tmp_path / "vl.parquet"
    pd.DataFrame(rows).to_parquet(f)
    ov = [f"data.train_files={f}", "data.train_batch_size=4", "data.max_prompt_length=96", "data.max_response_length=8",
          "data.image_min_pixels=64", "data.image_max_pixels=1024", "actor_rollout_ref.model.preset=tiny-qwen2-vl", "actor_rollout_ref.rollout.n=2",
          "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4",
          "actor_rollout_ref.actor.use_kl_loss=true", "actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=4",
          "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8", "actor_rollout_ref.rollout.max_num_seqs=16",
          "actor_rollout_ref.model.enable_gradient_checkpointing=false", "algorithm.adv_estimator=grpo", "reward.reward_manager=token_rule",
          "trainer.device=cpu", "trainer.val_before_train=false", "trainer.logger=[]", "trainer.n_gpus_per_node=1", "data.shuffle=false",
          "trainer.total_training_steps=1", f"trainer.default_local_dir={tmp_path}/ckpt", f"actor_rollout_ref.rollout.mode={mode}"]
    cfg = load_config("ppo_trainer", ov)
    from verl_b200.utils.tokenizer import ByteChatTokenizer

    tr = PPOTrainer(cfg, tokenizer=ByteChatTokenizer(), reward_fn=load_reward_manager(cfg, None), val_reward_fn=load_reward_manager(cfg, None))
    tr.init_workers()
    assert type(tr.actor_rollout_wg.worker.actor.engine.model).__name__ == "VisionLanguageModel"
    tr.global_steps = 1
    m = tr.step(next(iter(tr.train_dataloader)))
    b = tr._last_batch
    assert "multi_modal_inputs" in b.non_tensor_batch and (b.batch["input_ids"] == 2040).any()
    assert abs(m["actor/ppo_kl"]) < 1e-3 and m["actor/grad_norm"] >= 0      # (the gradient is zero when every group drew equal rewards)
    # rollout log-probs of the sampled tokens equal the trainer's recomputation
    d = ((b.batch["rollout_log_probs"] - b.batch["old_log_probs"]).abs() * b.batch["response_mask"]).max()
    assert d < 1e-3, d


def test_qwen2_5_vl_tower_and_logits_match_hf():
    """The windowed tower variant (RMSNorm, gated MLP, window attention with full-attention blocks) against Hugging Face
    Qwen2.5-VL: tower output for images whose grids are ragged against the window, and the logits of a sequence."""
    try:
        from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    except ImportError:
        pytest.skip("this transformers build has no Qwen2.5-VL")
    torch.manual_seed(0)
    hf_cfg = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, rope_theta=10000.0, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]},
                         tie_word_embeddings=False),
        vision_config=dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4, temporal_patch_size=2,
                           spatial_merge_size=2, window_size=16, out_hidden_size=64, fullatt_block_indexes=[1]),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503)
    hf = Qwen2_5_VLForConditionalGeneration(hf_cfg).float().eval()
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    assert cfg.vision["variant"] == "qwen2_5_vl" and cfg.vision["embed_dim"] == 32 and cfg.vision["hidden_size"] == 64 and cfg.hidden_size == 64
    cfg = cfg.replace(torch_dtype="float32", rms_norm_eps=hf_cfg.text_config.rms_norm_eps)
    ours = VisionLanguageModel(cfg, dtype=torch.float32, device=torch.device("cpu"))
    ours.load_hf_state_dict(hf.state_dict())
    ours.eval()
    g = torch.Generator().manual_seed(1)
    grid = torch.tensor([[1, 6, 10], [1, 4, 4], [1, 2, 6]])          # window = 2×2 merge groups: ragged, exact and narrower grids
    pixels = torch.randn(int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum()), 96, generator=g)
    with torch.no_grad():
        want = hf.model.visual(pixels, grid_thw=grid)
        want = want.pooler_output if hasattr(want, "pooler_output") else want
        got = ours.visual(pixels, grid)
    if isinstance(want, (tuple, list)):
        want = torch.cat(list(want), 0)
    assert got.shape == want.shape == (15 + 4 + 3, 64)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), (got - want).abs().max()
    text = lambda n: torch.randint(1, 400, (n,), generator=g).tolist()
    ids = torch.tensor(text(3) + [502] + [500] * 15 + [503] + text(4) + [502] + [500] * 4 + [503] + [502] + [500] * 3 + [503] + text(5))
    pos3, _ = get_rope_index(ids, grid, ours.vcfg)
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=torch.ones_like(ids)[None],
                  position_ids=pos3[:, None].contiguous()).logits[0]
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        got = ours(pb, pixel_values=pixels, image_grid_thw=grid, mrope_positions=pos3, return_logits=True)["logits"]
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()
    # config round trip in the newer layout
    back = ModelConfig.from_hf_dict(cfg.to_hf_dict())
    assert back.vision == cfg.vision


def test_sft_dataset_with_images():
    """Multi-turn SFT rows with images: ``<image>`` marks become placeholder runs of the image's size, only assistant tokens are
    targets, positions follow the image grid."""
    import numpy as np
    from PIL import Image

    from verl_b200.utils.dataset.sft_dataset import MultiTurnSFTDataset
    from verl_b200.utils.tokenizer import ByteChatTokenizer

    img = Image.fromarray(np.random.default_rng(0).integers(0, 255, (16, 24, 3), dtype=np.uint8))
    rows = [{"messages": [{"role": "user", "content": "describe <image> please"}, {"role": "assistant", "content": "a cat"}], "tools": None, "images": [img]},
            {"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}], "tools": None, "images": None}]
    vision = dict(patch_size=4, temporal_patch_size=2, spatial_merge_size=2, image_token_id=2040, vision_start_token_id=2042, mrope_section=[4, 6, 6])
    ds = MultiTurnSFTDataset(tokenizer=ByteChatTokenizer(), max_length=96, rows=rows, vision=vision, image_min_pixels=64, image_max_pixels=1024)
    a, b = ds[0], ds[1]
    g = a["multi_modal_inputs"]["image_grid_thw"]
    n = int(g[0, 1] * g[0, 2]) // 4
    ids = a["input_ids"][a["attention_mask"].bool()]
    run = (ids == 2040).nonzero().flatten()
    assert len(run) == n and int(run[-1] - run[0]) == n - 1 and int(ids[run[0] - 1]) == 2042 and int(ids[run[-1] + 1]) == 2043
    assert a["multi_modal_inputs"]["pixel_values"].shape == (int(g[0, 1] * g[0, 2]), 96)
    assert int(a["loss_mask"][run[0] - 1:run[-1] + 1].sum()) == 0 and int(a["loss_mask"].sum()) > 0      # image tokens are never targets
    assert a["position_ids"].shape == (4, 96) and b["multi_modal_inputs"] == {}
    live = b["attention_mask"].bool()
    assert torch.equal(b["position_ids"][0][live], b["position_ids"][3][live])
    # the text-only dataset is unchanged by the new arguments
    plain = MultiTurnSFTDataset(tokenizer=ByteChatTokenizer(), max_length=96, rows=rows[1:])
    assert torch.equal(plain[0]["input_ids"], b["input_ids"]) and plain[0]["position_ids"].dim() == 1


def test_qwen3_vl_tower_deepstack_and_logits_match_hf():
    """The Qwen3-VL family against Hugging Face: tower (interpolated learned positions, biased patch embedding, tanh-GELU MLP), the
    deep-stack features added to the decoder's stream after its first layers, the interleaved multimodal rotary embedding and the
    Qwen3 decoder (per-head q/k norms) — compared on the tower output, the deep-stack features and the logits of a sequence."""
    try:
        from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    except ImportError:
        pytest.skip("this transformers build has no Qwen3-VL")
    torch.manual_seed(0)
    hf_cfg = Qwen3VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                         head_dim=16, max_position_embeddings=512, rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                                                                     "mrope_section": [4, 2, 2], "mrope_interleaved": True},
                         tie_word_embeddings=False),
        vision_config=dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4, temporal_patch_size=2,
                           spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=36, deepstack_visual_indexes=[0, 2]),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503)
    hf = Qwen3VLForConditionalGeneration(hf_cfg).float().eval()
    with torch.no_grad():      # biases and norms away from their init values, so that a dropped one shows
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    v = cfg.vision
    assert v["variant"] == "qwen3_vl" and v["embed_dim"] == 32 and v["hidden_size"] == 64 and v["deepstack_visual_indexes"] == [0, 2]
    assert v["mrope_interleaved"] and v["mrope_section"] == [4, 2, 2] and cfg.qk_norm and not cfg.attention_bias and cfg.head_dim == 16
    cfg = cfg.replace(torch_dtype="float32", rms_norm_eps=hf_cfg.text_config.rms_norm_eps)
    ours = VisionLanguageModel(cfg, dtype=torch.float32, device=torch.device("cpu"))
    ours.load_hf_state_dict(hf.state_dict())
    ours.eval()
    g = torch.Generator().manual_seed(1)
    grid = torch.tensor([[1, 6, 10], [1, 4, 4], [1, 2, 6]])
    pixels = torch.randn(int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum()), 96, generator=g)
    with torch.no_grad():
        want = hf.model.visual(pixels, grid_thw=grid)
        got = ours.visual(pixels, grid)
    assert got.shape == want.pooler_output.shape == (15 + 4 + 3, 64)
    assert torch.allclose(got, want.pooler_output, atol=1e-5, rtol=1e-4), (got - want.pooler_output).abs().max()
    assert len(ours.visual.last_deepstack) == 2
    for a, b in zip(ours.visual.last_deepstack, want.deepstack_features):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4), (a - b).abs().max()
    text = lambda n: torch.randint(1, 400, (n,), generator=g).tolist()
    ids = torch.tensor(text(3) + [502] + [500] * 15 + [503] + text(4) + [502] + [500] * 4 + [503] + [502] + [500] * 3 + [503] + text(5))
    pos3, _ = get_rope_index(ids, grid, ours.vcfg)
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=torch.ones_like(ids)[None],
                  position_ids=pos3[:, None].contiguous()).logits[0]
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        got = ours(pb, pixel_values=pixels, image_grid_thw=grid, mrope_positions=pos3, return_logits=True)["logits"]
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()
    # the deep-stack path matters: without it the logits differ
    with torch.no_grad():
        ours.visual.deepstack_merger_list[0].linear_fc2.weight.zero_()
        ours.visual.deepstack_merger_list[0].linear_fc2.bias.zero_()
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        off = ours(pb, pixel_values=pixels, image_grid_thw=grid, mrope_positions=pos3, return_logits=True)["logits"]
    assert (off - want).abs().max() > 1e-3
    # names and config round trip in the family's layout
    names = {n for n, _ in ours.hf_named_tensors()}
    assert "model.visual.pos_embed.weight" in names and "model.visual.deepstack_merger_list.1.norm.bias" in names
    back = ModelConfig.from_hf_dict(cfg.to_hf_dict())
    assert back.vision == cfg.vision and back.qk_norm and back.head_dim == 16


def test_video_inputs_frames_to_patches_positions_and_tower():
    """Videos given as frames: patch layout (a video of identical frames repeats the image's patches per temporal patch), frame
    sampling and padding to the temporal patch size, the 3-stream positions of a prompt that mixes an image and a video against
    Hugging Face Qwen2.5-VL (temporal stream scaled by seconds-per-patch x tokens-per-second), and the tower on a t > 1 grid."""
    import numpy as np

    from verl_b200.utils.dataset.vision_utils import expand_visual_tokens, image_to_patches, process_video, video_to_patches

    rng = np.random.default_rng(0)
    frame = rng.integers(0, 255, (16, 24, 3), dtype=np.uint8)
    frames, sec = process_video([frame] * 3, factor=8, min_pixels=64, max_pixels=16 * 24)        # 3 frames -> padded to 4
    assert len(frames) == 4 and frames[0].size == (24, 16) and sec == 1.0
    pv, gv = video_to_patches(frames, 4, 2, 2)
    pi, gi = image_to_patches(frames[0], 4, 2, 2)
    assert gv.tolist() == [[2, 4, 6]] and gi.tolist() == [[1, 4, 6]] and torch.equal(pv[:24], pi) and torch.equal(pv[24:], pi)
    frames, sec = process_video({"frames": np.stack([frame] * 10), "fps": 5.0}, factor=8, min_pixels=64, max_pixels=16 * 24, fps=2.0)
    assert len(frames) == 4 and sec == 1.0                                                        # 2 s at 2 fps = 4 frames; 2 frames per patch
    frames, sec = process_video({"frames": [frame] * 10, "fps": 10.0, "nframes": 4}, factor=8, min_pixels=64, max_pixels=16 * 24)
    assert len(frames) == 4 and abs(sec - 2 / 4.0) < 1e-9                                         # 4 of 10 frames at 10 fps -> 4 fps
    assert expand_visual_tokens([1, 500, 2, 501, 3], torch.tensor([[1, 4, 4], [2, 4, 4]]), (500, 501)) == [1] + [500] * 4 + [2] + [501] * 8 + [3]
    try:
        from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    except ImportError:
        pytest.skip("this transformers build has no Qwen2.5-VL")
    torch.manual_seed(0)
    hf_cfg = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, rope_theta=10000.0, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
        vision_config=dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4, temporal_patch_size=2,
                           spatial_merge_size=2, window_size=16, out_hidden_size=64, fullatt_block_indexes=[1], tokens_per_second=2),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503)
    hf = Qwen2_5_VLForConditionalGeneration(hf_cfg).float().eval()
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict()).replace(torch_dtype="float32")
    assert cfg.vision["tokens_per_second"] == 2.0
    ours = VisionLanguageModel(cfg, dtype=torch.float32, device=torch.device("cpu"))
    ours.load_hf_state_dict(hf.state_dict())
    img_grid, vid_grid = torch.tensor([[1, 4, 4]]), torch.tensor([[3, 4, 8]])
    ids = torch.tensor([7, 8, 502] + [500] * 4 + [503, 9, 502] + [501] * 24 + [503, 10, 11])
    second_per_grid = 1.5                                                                          # e.g. 2 frames per patch sampled at 4/3 fps
    got, delta = get_rope_index(ids, torch.cat([img_grid, vid_grid]), ours.vcfg,
                                grid_t_scale=torch.tensor([1.0, second_per_grid * cfg.vision["tokens_per_second"]]))
    # the published rule (text continues from the largest position + 1; a video's temporal index is
    # floor(patch index x seconds per patch x tokens per second)), written out by hand for this prompt
    want = [(0, 0, 0), (1, 1, 1), (2, 2, 2), (3, 3, 3), (3, 3, 4), (3, 4, 3), (3, 4, 4), (5, 5, 5), (6, 6, 6), (7, 7, 7)]
    want += [(8 + 3 * t, 8 + h, 8 + w) for t in range(3) for h in range(2) for w in range(4)]
    want += [(15, 15, 15), (16, 16, 16), (17, 17, 17)]
    assert got.t().tolist() == [list(x) for x in want]
    assert delta == 18 - len(ids)
    pix = torch.randn(3 * 4 * 8, 96)
    with torch.no_grad():
        w = hf.model.visual(pix, grid_thw=vid_grid)
        w = w.pooler_output if hasattr(w, "pooler_output") else w
        g = ours.visual(pix, vid_grid)
    assert torch.allclose(g, w, atol=1e-5, rtol=1e-4)
