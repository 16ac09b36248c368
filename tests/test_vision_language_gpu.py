"""Vision-language model on the GPU kernels (bf16): engine log-probs and rollout greedy tokens against an fp32 copy of the
same weights run through plain PyTorch on the CPU."""

import pytest
import torch

from verl_b200.models.config import ModelConfig
from verl_b200.models.transformer import PackedBatch
from verl_b200.models.vision import VisionLanguageModel, get_rope_index

pytestmark = pytest.mark.gpu


def _cfg():
    return ModelConfig(model_type="qwen2", vocab_size=4096, hidden_size=512, intermediate_size=1536, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=128, rope_theta=1e4, max_position_embeddings=4096,
                       vision=dict(depth=2, embed_dim=64, num_heads=2, mlp_ratio=2.0, in_channels=3, patch_size=4, temporal_patch_size=2,
                                   spatial_merge_size=2, hidden_size=512, image_token_id=4000, video_token_id=4001, vision_start_token_id=4002,
                                   mrope_section=[16, 24, 24]))


def _batch(g):
    import numpy as np

    from verl_b200.protocol import DataProto

    P, R, bs = 48, 16, 4
    input_ids = torch.zeros(bs, P + R, dtype=torch.long)
    att = torch.zeros(bs, P + R, dtype=torch.long)
    mm = []
    for i, grid in enumerate([[[1, 4, 8]], [], [[1, 4, 4], [1, 2, 2]], [[1, 8, 8]]]):
        ids = []
        for t, h, w in grid:
            ids += [4002] + [4000] * (t * h * w // 4) + [4003]
        ids += torch.randint(1, 3900, (6 + i,), generator=g).tolist()
        n_patch = sum(t * h * w for t, h, w in grid)
        mm.append({"pixel_values": torch.randn(n_patch, 96, generator=g), "image_grid_thw": torch.tensor(grid).reshape(-1, 3)} if grid else {})
        resp = torch.randint(1, 3900, (R - 2 * i,), generator=g).tolist()
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
    return data, mm, P


def test_engine_log_probs_and_update_on_image_prompts():
    from tests.test_engine_on_cpu import loss_fn
    from verl_b200.ops import _ext
    from verl_b200.workers.engine.fsdp.engine import FSDPEngine

    eng = FSDPEngine(_cfg(), {"seed": 3}, {"lr": 1e-4, "clip_grad": 1.0}, {})
    eng.initialize()
    assert eng.store.flat.is_cuda and eng.store.flat.dtype == torch.bfloat16
    ref = VisionLanguageModel(_cfg(), dtype=torch.float32, device=torch.device("cpu"), seed=3)
    ref.load_state_dict({k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()})
    g = torch.Generator().manual_seed(5)
    data, mm, P = _batch(g)
    lp = eng.infer_batch(data)["model_output"]["log_probs"].cpu()
    b = data.batch
    worst = 0.0
    for i in range(len(mm)):
        m = b["attention_mask"][i].bool()
        ids = b["input_ids"][i][m]
        grid = mm[i].get("image_grid_thw")
        pos3, _ = get_rope_index(ids, grid, ref.vcfg)
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        with torch.no_grad():
            logits = ref(pb, pixel_values=mm[i].get("pixel_values"), image_grid_thw=grid, mrope_positions=pos3, return_logits=True)["logits"]
        want = torch.log_softmax(logits, -1)
        n_prompt = int(b["attention_mask"][i, :P].sum())
        for t in range(int(b["attention_mask"][i, P:].sum())):
            worst = max(worst, abs(float(lp[i, t]) - float(want[n_prompt - 1 + t, ids[n_prompt + t]])))
    assert worst < 0.08, worst
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(data, loss_fn)
    assert eng.model.visual.patch_embed.proj.weight.main_grad.abs().sum() > 0
    gn = eng.optimizer_step()
    torch.cuda.synchronize()
    _ext.check_status("vision-language engine")
    assert gn == gn and gn > 0


def test_rollout_greedy_tokens_with_images():
    from verl_b200.ops import _ext
    from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams

    model = VisionLanguageModel(_cfg(), dtype=torch.bfloat16, device=torch.device("cuda"), seed=11).eval()
    ref = VisionLanguageModel(_cfg(), dtype=torch.float32, device=torch.device("cpu"), seed=11).eval()
    ref.load_state_dict({k: v.detach().float().cpu() for k, v in model.state_dict().items()})
    g = torch.Generator().manual_seed(2)
    grid = torch.tensor([[1, 4, 8]])
    prompt = [7, 8, 4002] + [4000] * 8 + [4003, 9, 10, 11]
    mm = {"pixel_values": torch.randn(32, 96, generator=g), "image_grid_thw": grid}
    eng = InferenceEngine(model, max_num_seqs=8, max_model_len=128, num_blocks=64)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, logprobs=True)
    outs = eng.generate([prompt, [5, 6, 7, 8, 9]], sp, multi_modal=[mm, None])
    torch.cuda.synchronize()
    _ext.check_status("vision-language rollout")
    # teacher-forced check: the fp32 model gives each generated token a log-prob close to the rollout's own
    for o, (p, m) in zip(outs, [(prompt, mm), ([5, 6, 7, 8, 9], None)]):
        ids = torch.tensor(list(p) + list(o.token_ids))
        pos3, _ = get_rope_index(ids, m["image_grid_thw"] if m else None, ref.vcfg)
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        with torch.no_grad():
            logits = ref(pb, pixel_values=m["pixel_values"] if m else None, image_grid_thw=m["image_grid_thw"] if m else None,
                         mrope_positions=pos3, return_logits=True)["logits"]
        want = torch.log_softmax(logits, -1)
        for j, (tok, lp) in enumerate(zip(o.token_ids, o.log_probs)):
            assert abs(float(want[len(p) - 1 + j, tok]) - lp) < 0.1, (j, float(want[len(p) - 1 + j, tok]), lp)
