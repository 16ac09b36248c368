"""Rollout engine and prefix-shared training pass on the GPU kernels (tcgen05 GEMMs, paged decode, CUDA-graph decode)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(seed=0):
    from verl_b200.models.config import PRESETS
    from verl_b200.models.transformer import DecoderLM

    return DecoderLM(PRESETS["tiny-qwen2-gpu"], dtype=torch.bfloat16, device="cuda", seed=seed)


def test_rollout_log_probs_match_a_training_forward_and_fp8_mode_stays_close():
    from verl_b200.models.transformer import PackedBatch
    from verl_b200.ops import _ext
    from verl_b200.workers.rollout import InferenceEngine, SamplingParams

    model = _model()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(10, model.cfg.vocab_size, (int(n),), generator=g).tolist() for n in (33, 70, 129, 18)]
    sp = SamplingParams(temperature=1.0, max_tokens=24, seed=3, top_logprobs=4)
    eng = InferenceEngine(model, max_num_seqs=8, max_model_len=256, num_blocks=64, sync_interval=4)
    outs = eng.generate(prompts, sp)
    assert eng._graph is not None                                  # the decode step ran as a CUDA graph
    worst = 0.0
    for p, o in zip(prompts, outs):
        ids = torch.tensor(p + o.token_ids, device="cuda")
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32, device="cuda"), torch.tensor([0, len(ids)], dtype=torch.int32, device="cuda"))
        with torch.no_grad():
            lp = torch.log_softmax(model(pb, return_logits=True)["logits"].float(), -1)
        want = lp[len(p) - 1: len(ids) - 1].gather(1, ids[len(p):, None])[:, 0]
        got = torch.tensor(o.log_probs, device="cuda")
        worst = max(worst, (want - got).abs().max().item())
        top = torch.tensor(o.top_log_probs, device="cuda")
        assert top.shape == (24, 4) and (top[:, 0] >= top[:, 1]).all() and (got <= top[:, 0] + 1e-4).all()
        ref_top = lp[len(p) - 1: len(ids) - 1].topk(4, -1).values
        assert (ref_top - top).abs().max() < 0.08
    assert worst < 0.08, worst                                     # bf16 decode path vs bf16 packed forward
    eng.sleep()

    # W8A8 rollout: same sampler seed, log-probs of ITS tokens re-scored by the bf16 model stay close
    for quant in ("fp8", "fp8_block"):
        eng8 = InferenceEngine(model, max_num_seqs=8, max_model_len=256, num_blocks=64, sync_interval=4, quantization=quant)
        outs8 = eng8.generate(prompts, SamplingParams(temperature=1.0, max_tokens=24, seed=3))
        assert len(eng8._w8) == 4 * model.cfg.num_hidden_layers
        diffs = []
        for p, o in zip(prompts, outs8):
            ids = torch.tensor(p + o.token_ids, device="cuda")
            pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32, device="cuda"), torch.tensor([0, len(ids)], dtype=torch.int32, device="cuda"))
            with torch.no_grad():
                lp = torch.log_softmax(model(pb, return_logits=True)["logits"].float(), -1)
            want = lp[len(p) - 1: len(ids) - 1].gather(1, ids[len(p):, None])[:, 0]
            diffs.append((want - torch.tensor(o.log_probs, device="cuda")).abs())
        d = torch.cat(diffs)
        assert d.mean() < 0.1 and d.max() < 1.0, (quant, d.mean().item(), d.max().item())
        eng8.sleep()
        assert not eng8._w8
    torch.cuda.synchronize()
    _ext.check_status("rollout engine test")


def test_prefix_shared_training_pass_matches_plain_pass_on_gpu():
    from verl_b200.models.config import PRESETS
    from verl_b200.ops import _ext
    from verl_b200.protocol import DataProto
    from verl_b200.workers.engine.fsdp.engine import FSDPEngine
    from verl_b200.workers.utils.losses import ppo_loss

    cfg = {"clip_ratio": 0.2, "use_kl_loss": True, "kl_loss_coef": 1e-3, "entropy_coeff": 0.0, "loss_agg_mode": "token-mean"}

    def batch(**meta):
        g = torch.Generator().manual_seed(0)
        n_prompts, n, P, R, V = 4, 8, 200, 150, 4096
        bs = n_prompts * n
        prompts = torch.randint(10, V, (n_prompts, P), generator=g)
        patt = torch.ones(n_prompts, P, dtype=torch.int64)
        for i in range(n_prompts):
            patt[i, : 17 * i] = 0
        ids = torch.cat([prompts.repeat_interleave(n, 0), torch.randint(10, V, (bs, R), generator=g)], 1)
        att = torch.cat([patt.repeat_interleave(n, 0), torch.ones(bs, R, dtype=torch.int64)], 1)
        for i in range(bs):
            att[i, P + R - (i % 5) * 11:] = 0
        pos = torch.clip(torch.cumsum(att, -1) - 1, min=0)
        m = {"use_dynamic_bsz": True, "max_token_len_per_gpu": 4096, "temperature": 1.0, "calculate_entropy": True}
        m.update(meta)
        return DataProto.from_dict(tensors={
            "input_ids": ids, "attention_mask": att, "position_ids": pos, "responses": ids[:, -R:], "response_mask": att[:, -R:],
            "old_log_probs": torch.full((bs, R), -8.3), "ref_log_prob": torch.full((bs, R), -8.3),
            "advantages": torch.randn(bs, R, generator=g)}, meta_info=m)

    res = []
    for meta in ({}, {"use_prefix_grouper": True}):
        eng = FSDPEngine(PRESETS["tiny-qwen2-gpu"], {"seed": 1}, {"lr": 1e-4}, {})
        eng.initialize()
        data = batch(**meta)
        lp = eng.infer_batch(data)["model_output"]["log_probs"]
        eng.optimizer_zero_grad()
        eng.forward_backward_batch(data, lambda model_output, data, dp_group=None: ppo_loss(cfg, model_output, data))
        res.append((lp.float().cpu(), eng.store.grad.float().cpu().clone()))
    (lp0, g0), (lp1, g1) = res
    assert (lp0 - lp1).abs().max() < 0.06, (lp0 - lp1).abs().max()
    cos = torch.nn.functional.cosine_similarity(g0.flatten(), g1.flatten(), dim=0).item()
    assert cos > 0.995, cos
    assert abs(g0.norm() / g1.norm() - 1) < 0.03
    torch.cuda.synchronize()
    _ext.check_status("prefix sharing on gpu")


def test_chunked_prefill_and_prefix_cache_give_the_log_probs_of_a_plain_prefill():
    """Prompts of 300-700 tokens under a 256-token step budget are prefilled in chunks that attend to the chunks already in
    the paged cache (q_starts > 128: the kernels skip whole query tiles); a second call reuses the cached blocks of the first.
    Sampled tokens are seeded identically, so the token ids must agree with the unchunked engine while the log-probs agree to
    bf16 accuracy."""
    from verl_b200.ops import _ext
    from verl_b200.workers.rollout import InferenceEngine, SamplingParams

    model = _model(2)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(10, model.cfg.vocab_size, (int(n),), generator=g).tolist() for n in (700, 300, 45, 513)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, seed=3)
    plain = InferenceEngine(model, max_num_seqs=8, max_model_len=1024, num_blocks=96, sync_interval=4, max_num_batched_tokens=8192,
                            enable_prefix_caching=False)
    want = plain.generate(prompts, sp)
    plain.sleep()
    eng = InferenceEngine(model, max_num_seqs=8, max_model_len=1024, num_blocks=96, sync_interval=4, max_num_batched_tokens=256)
    got = eng.generate(prompts, sp)
    assert eng.stats["prefill_chunks"] == 2 + 1 + 0 + 2

    def close(a, b):
        # greedy decoding on bf16 logits: a near-tie may flip a token, after which the continuations differ legitimately
        n = next((i for i, (x, y) in enumerate(zip(a.token_ids, b.token_ids)) if x != y), len(a.token_ids))
        assert n >= 4, (a.token_ids, b.token_ids)
        d = max(abs(x - y) for x, y in zip(a.log_probs[:n], b.log_probs[:n]))
        assert d < 0.08, d

    for a, b in zip(got, want):
        close(a, b)
    # follow-up turns inside the same wake period hit the cached blocks (prompt and generated tokens)
    turn2 = [p + o.token_ids + [21, 22, 23] for p, o in zip(prompts[:2], got[:2])]
    hits0 = eng.stats["prefix_cache_hit_tokens"]
    got2 = eng.generate(turn2, sp)
    assert eng.stats["prefix_cache_hit_tokens"] - hits0 == (711 // 64) * 64 + (311 // 64) * 64
    eng.sleep()
    plain.wake_up()
    want2 = plain.generate(turn2, sp)
    for a, b in zip(got2, want2):
        close(a, b)
    torch.cuda.synchronize()
    _ext.check_status("chunked prefill")


def test_activation_offload_keeps_gradients_and_moves_the_saved_tensors_to_the_host():
    """`model.enable_activation_offload`: what autograd saves inside the decoder layers is copied to pinned host memory and brought
    back for backward; gradients and the gradient norm equal the plain run."""
    from tests.test_engine_on_cpu import loss_fn, make_batch
    from verl_b200.workers.engine.fsdp.engine import FSDPEngine

    res = {}
    for off in (False, "again", True):
        eng = FSDPEngine({"preset": "tiny-qwen2-gpu", "enable_activation_offload": off is True, "activation_offload_min_numel": 4096}, {"seed": 1},
                         {"lr": 1e-3, "clip_grad": 1.0}, {})
        eng.initialize()
        data = make_batch(bs=8, P=70, R=90, vocab=4096)
        data.meta_info["micro_batch_size_per_gpu"] = 4
        eng.optimizer_zero_grad()
        eng.forward_backward_batch(data, loss_fn)
        torch.cuda.synchronize()
        res[off] = (eng.store.grad.clone(), eng.optimizer_step())
        if off is True:
            assert eng.model._activation_offloader.bytes_offloaded > 1 << 20
    # two plain runs are bit-identical; the offloaded run hands backward fresh, aligned copies of the saved tensors, which may take
    # another GEMM path than a view of a larger buffer does, so it agrees to bf16 rounding, with the same gradient norm. That the
    # copies themselves are exact is checked tensor by tensor in the next test.
    noise = ((res["again"][0] - res[False][0]).norm() / res[False][0].norm()).item()
    rel = ((res[True][0] - res[False][0]).norm() / res[False][0].norm()).item()
    assert noise < 1e-6 and rel < 5e-3, (rel, noise)
    assert abs(res[True][1] - res[False][1]) < 1e-4 * res[False][1], (res[True][1], res[False][1])


def test_activation_offload_round_trip_is_bit_exact_and_ordered():
    """Every tensor saved under the hooks comes back with exactly its bytes, whatever the order backward asks for them in, and
    small / non-contiguous / parameter tensors are left on the device."""
    from verl_b200.utils.activation_offload import ActivationOffloader

    off = ActivationOffloader(min_numel=1024, prefetch=True)
    g = torch.Generator(device="cuda").manual_seed(3)
    src = [torch.randn(257, 129, device="cuda", generator=g).to(dt) for dt in (torch.bfloat16, torch.float32, torch.bfloat16, torch.float16)]
    small = torch.randn(8, device="cuda")
    strided = torch.randn(64, 64, device="cuda").t()
    par = torch.nn.Parameter(torch.randn(64, 64, device="cuda"))
    keep = [t.clone() for t in src]
    packed = [off.pack(t) for t in src]
    assert all(isinstance(p, tuple) for p in packed)
    assert off.pack(small) is small and off.pack(strided) is strided and off.pack(par) is par
    off.stream.synchronize()
    for t in src:                                     # once the copies have landed the device originals may be overwritten
        t.zero_()
    for i in (3, 2, 0, 1):                            # backward order, then out of order
        back = off.unpack(packed[i])
        assert back.is_cuda and back.dtype == keep[i].dtype and torch.equal(back, keep[i])
    assert off.bytes_offloaded == sum(t.numel() * t.element_size() for t in keep)
    assert off.unpack(small) is small
