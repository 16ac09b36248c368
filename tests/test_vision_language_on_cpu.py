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
