import numpy as np
import pytest
import torch

from verl_b200.models.config import PRESETS
from verl_b200.models.transformer import DecoderLM, PackedBatch
from verl_b200.workers.rollout import InferenceEngine, SamplingParams
from verl_b200.workers.rollout.engine import _sample_reference
from verl_b200.workers.rollout.scheduler import STEP_DECODE, STEP_IDLE, STEP_PREFILL, Scheduler


def greedy_oracle(model, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        t = torch.tensor(ids)
        pb = PackedBatch(t, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        with torch.no_grad():
            ids.append(int(model(pb, return_logits=True)["logits"][-1].argmax()))
    return ids[len(prompt):]


@pytest.fixture(scope="module")
def model():
    return DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=3)


def test_scheduler_prefill_decode_and_limits():
    s = Scheduler(num_blocks=9, block_size=64, max_num_seqs=4, max_batched_tokens=1024)
    s.add(0, 100, 10)
    s.add(1, 60, 10)
    kind, ids, slots, lens, forks = s.step()
    assert kind == STEP_PREFILL and ids.tolist() == [0, 1] and lens.tolist() == [100, 60] and (forks < 0).all()
    assert len(s.blocks(0)) == 2 and len(s.blocks(1)) == 1
    kind, ids, slots, lens, _ = s.step()
    assert kind == STEP_DECODE and lens.tolist() == [101, 61]
    for _ in range(4):
        s.step()
    assert len(s.blocks(1)) == 2          # crossed a block boundary at 65 tokens
    s.finish(0)
    s.finish(1)
    assert s.step()[0] == STEP_IDLE and s.num_free_blocks == 8
    with pytest.raises(ValueError):
        s.add(5, 64 * 9, 1)               # can never fit


def test_scheduler_fork_shares_prompt_blocks():
    s = Scheduler(num_blocks=16, block_size=64, max_num_seqs=8, max_batched_tokens=4096)
    for i in range(3):
        s.add(i, 150, 20, share_key=77)
    kind, ids, slots, lens, forks = s.step()
    assert kind == STEP_PREFILL and forks.tolist() == [-1, 0, 0]
    b0, b1, b2 = s.blocks(0), s.blocks(1), s.blocks(2)
    assert b0[:2].tolist() == b1[:2].tolist() == b2[:2].tolist()    # two full blocks shared
    assert len({int(b0[2]), int(b1[2]), int(b2[2])}) == 3            # private partial blocks
    for i in range(3):
        s.finish(i)
    assert s.num_free_blocks == 15


def test_scheduler_preempts_newest_when_out_of_blocks():
    s = Scheduler(num_blocks=4, block_size=64, max_num_seqs=4, max_batched_tokens=4096)   # 3 usable blocks
    s.add(0, 60, 100)
    s.add(1, 60, 100)
    kind, ids, *_ = s.step()
    assert kind == STEP_PREFILL and ids.tolist() == [0, 1]        # one block each, one block left
    seen_preempt = False
    for _ in range(12):
        kind, ids, slots, lens, _f = s.step()
        if s.num_preemptions > 0:
            seen_preempt = True
            break
    assert seen_preempt and ids.tolist() == [0]                    # the newest sequence (1) was evicted
    assert s.num_waiting == 1 and s.num_preempted(1) == 1
    s.finish(0)
    kind, ids, slots, lens, _f = s.step()
    assert kind == STEP_PREFILL and ids.tolist() == [1] and lens[0] > 60   # recompute prompt + generated tokens


def test_generate_matches_greedy_oracle_with_forks(model):
    eng = InferenceEngine(model, max_num_seqs=8, max_model_len=128, num_blocks=16, sync_interval=4)
    g = torch.Generator().manual_seed(0)
    base = [torch.randint(10, 2048, (n,), generator=g).tolist() for n in (20, 33)]
    prompts = [base[0], base[0], base[1], base[1], base[0]]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    assert eng.stats["forked"] == 3
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_oracle(model, p, 12)
        assert o.stop_reason == "length" and len(o.log_probs) == 12 and all(lp <= 0 for lp in o.log_probs)


def test_generate_with_preemption_still_matches(model):
    # 3 blocks of 64 tokens for two sequences that each grow to 70+ tokens forces a recompute preemption
    eng = InferenceEngine(model, max_num_seqs=4, max_model_len=128, num_blocks=4, sync_interval=2, enable_prefix_sharing=False)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(10, 2048, (50,), generator=g).tolist() for _ in range(2)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=30))
    assert eng.sched.num_preemptions >= 1
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_oracle(model, p, 30)


def test_eos_stops_generation(model):
    eng = InferenceEngine(model, max_num_seqs=4, max_model_len=128, num_blocks=8, sync_interval=4)
    p = list(range(10, 30))
    ref = greedy_oracle(model, p, 10)
    eos = ref[4]
    first = ref.index(eos)
    out = eng.generate([p], SamplingParams(temperature=0.0, max_tokens=10), eos_token_id=eos)[0]
    assert out.token_ids == ref[: first + 1] and out.stop_reason == "stop"


def test_sleep_and_wake(model):
    eng = InferenceEngine(model, max_num_seqs=2, max_model_len=64, num_blocks=4)
    eng.wake_up()
    assert eng.cache is not None
    eng.sleep()
    assert eng.cache is None
    out = eng.generate([[11, 12, 13]], SamplingParams(temperature=0.0, max_tokens=3))
    assert len(out[0].token_ids) == 3


def test_sampling_reference_topk_topp():
    g = torch.Generator().manual_seed(0)
    logits = torch.tensor([[5.0, 4.0, 1.0, 0.0, -1.0]]).repeat(200, 1)
    tok, lp = _sample_reference(logits, 1.0, 2, 1.0, g)
    assert set(tok.tolist()) <= {0, 1}
    tok, _ = _sample_reference(logits, 1.0, -1, 0.5, g)
    assert set(tok.tolist()) == {0}
    tok, lp = _sample_reference(logits, 0.0, -1, 1.0, g)
    assert tok.tolist() == [0] * 200


def test_rollout_records_the_routed_experts_of_every_fed_token():
    """Router replay R3: with ``record_routing`` the engine returns, per sequence, the experts chosen for every token of
    prompt + response in every layer. They must equal what a plain forward pass of the same model chooses for those tokens
    (siblings that share a prompt's KV blocks share its routing rows), and forcing them reproduces the same log-probs."""
    import numpy as np

    from verl_b200.models.config import PRESETS
    from verl_b200.models.transformer import DecoderLM, PackedBatch
    from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams

    cfg = PRESETS["tiny-qwen3-moe"]
    model = DecoderLM(cfg, dtype=torch.float32, seed=5)
    eng = InferenceEngine(model, max_num_seqs=8, max_model_len=96, num_blocks=24, sync_interval=4)
    eng.record_routing = True
    g = torch.Generator().manual_seed(0)
    base = [torch.randint(10, 2000, (int(n),), generator=g).tolist() for n in (9, 17, 30)]
    prompts = [base[0], base[0], base[1], base[2], base[2]]          # two groups of siblings
    outs = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=7, seed=3))
    L, k = cfg.num_hidden_layers, cfg.num_experts_per_tok
    for p, o in zip(prompts, outs):
        ids = p + o.token_ids
        rt = o.routed_experts
        assert rt is not None and rt.shape == (len(ids), L, k) and rt.dtype == np.int16
        pb = PackedBatch(torch.tensor(ids), torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        for layer in model.layers:
            layer.mlp.record_routing = True
        with torch.no_grad():
            model.forward_hidden(pb)
        want = torch.stack([layer.mlp.last_topk for layer in model.layers], 1).numpy()
        fed = len(ids) - 1                                         # the last sampled token was never fed to the model
        assert (np.sort(rt[:fed], -1) == np.sort(want[:fed], -1)).all()
        # forcing the recorded routing gives the rollout's log-probs back
        pb.routed_experts = torch.from_numpy(rt.astype(np.int64))
        with torch.no_grad():
            lp = model(pb, labels=torch.roll(torch.tensor(ids), -1), need_entropy=False)["log_probs"]
        got = lp[len(p) - 1:len(ids) - 1]
        assert torch.allclose(got, torch.tensor(o.log_probs), atol=1e-4)


def test_scheduler_chunks_a_prompt_longer_than_the_step_budget():
    s = Scheduler(num_blocks=16, block_size=64, max_num_seqs=4, max_batched_tokens=128, prefix_caching=False)
    s.add(0, 300, 5, tokens=list(range(300)))
    s.add(1, 40, 5, tokens=list(range(1000, 1040)))
    seen = []
    for _ in range(3):
        kind, ids, slots, lens, forks = s.step()
        assert kind == STEP_PREFILL
        seen.append((ids.tolist(), s.starts.tolist(), lens.tolist()))
    # 128 + 128 + 44 tokens of sequence 0; the short one joins the last chunk's step with the budget that is left
    assert seen == [([0], [0], [128]), ([0], [128], [128]), ([0, 1], [256, 0], [44, 40])]
    assert s.extra_prefill_chunks == 2 and s.num_running == 2
    kind, ids, slots, lens, _ = s.step()
    assert kind == STEP_DECODE and ids.tolist() == [0, 1] and lens.tolist() == [301, 41]
    # with chunking off the long prompt is one oversized step, as before
    s2 = Scheduler(num_blocks=16, block_size=64, max_num_seqs=4, max_batched_tokens=128, chunked_prefill=False)
    s2.add(0, 300, 5)
    kind, ids, slots, lens, _ = s2.step()
    assert kind == STEP_PREFILL and lens.tolist() == [300] and s2.starts.tolist() == [0]


def test_scheduler_prefix_cache_hits_eviction_and_generated_blocks():
    s = Scheduler(num_blocks=8, block_size=64, max_num_seqs=4, max_batched_tokens=4096)          # 7 usable blocks
    sys_prompt = list(range(500, 500 + 128))
    a = sys_prompt + [7] * 30
    s.add(0, len(a), 50, tokens=a)
    kind, ids, slots, lens, _ = s.step()
    assert kind == STEP_PREFILL and s.starts.tolist() == [0] and lens.tolist() == [158]
    for _ in range(41):                                    # decode steps: 199 tokens have KV afterwards
        s.step()
    blocks_a = s.blocks(0)
    gen = [9] * 40
    s.finish(0, tokens=a + gen)                            # 198 tokens: three full blocks stay findable, nothing is "free" yet
    assert s.num_free_blocks == 7
    # same system prompt, different tail: the two shared blocks are reused, 20 + the tail is computed
    b = sys_prompt + [8] * 20
    s.add(1, len(b), 10, tokens=b)
    kind, ids, slots, lens, _ = s.step()
    assert s.starts.tolist() == [128] and lens.tolist() == [20] and s.blocks(1)[:2].tolist() == blocks_a[:2].tolist()
    # the next turn of the first conversation: prompt + generated tokens + new user text; generated blocks hit too
    c = a + gen + [5] * 10
    s.add(2, len(c), 10, tokens=c)
    kind, ids, slots, lens, _ = s.step()
    assert s.starts.tolist() == [192] and lens.tolist() == [len(c) - 192] and s.blocks(2)[:3].tolist() == blocks_a[:3].tolist()
    assert s.prefix_cache_hit_tokens == 128 + 192
    s.finish(1)
    s.finish(2)
    # an identical prompt never hits on its last token: one token at least is computed
    d = sys_prompt
    s.add(3, len(d), 4, tokens=d)
    kind, ids, slots, lens, _ = s.step()
    assert s.starts.tolist() == [64] and lens.tolist() == [64]
    s.finish(3)
    # pressure: unused cached blocks are handed out again (oldest first) and stop being findable
    big = list(range(3000, 3000 + 64 * 6))
    s.add(4, len(big), 10, tokens=big)
    kind, ids, slots, lens, _ = s.step()
    assert kind == STEP_PREFILL and s.starts.tolist() == [0]
    s.finish(4)
    s.add(5, len(a), 10, tokens=a)
    s.step()
    assert s.starts.tolist() == [0]                        # the system prompt's blocks were recycled


def test_engine_chunked_prefill_and_prefix_cache_match_the_oracle(model):
    g = torch.Generator().manual_seed(7)
    long_p = torch.randint(10, 2048, (150,), generator=g).tolist()
    short_p = torch.randint(10, 2048, (20,), generator=g).tolist()
    eng = InferenceEngine(model, max_num_seqs=4, max_model_len=256, num_blocks=24, sync_interval=4, max_num_batched_tokens=64)
    outs = eng.generate([long_p, short_p], SamplingParams(temperature=0.0, max_tokens=8))
    assert eng.stats["prefill_chunks"] == 2                # 64 + 64 + 22
    assert outs[0].token_ids == greedy_oracle(model, long_p, 8) and outs[1].token_ids == greedy_oracle(model, short_p, 8)
    # second call inside the same wake period: a follow-up turn reuses the first conversation's blocks (prompt AND response)
    turn2 = long_p + outs[0].token_ids + [33, 34, 35]
    other = long_p[:128] + [77] * 9
    before = eng.stats["prefill_tokens"]
    outs2 = eng.generate([turn2, other], SamplingParams(temperature=0.0, max_tokens=6))
    assert eng.stats["prefix_cache_hit_tokens"] == 128 + 128          # two full blocks each (150 + 7 fed tokens < 3 blocks)
    assert eng.stats["prefill_tokens"] - before == (len(turn2) - 128) + (len(other) - 128)
    assert outs2[0].token_ids == greedy_oracle(model, turn2, 6) and outs2[1].token_ids == greedy_oracle(model, other, 6)
    # with both features off the same requests give the same tokens in single oversized steps
    eng0 = InferenceEngine(model, max_num_seqs=4, max_model_len=256, num_blocks=24, sync_interval=4, max_num_batched_tokens=64,
                           enable_chunked_prefill=False, enable_prefix_caching=False)
    outs0 = eng0.generate([long_p, short_p], SamplingParams(temperature=0.0, max_tokens=8))
    assert [o.token_ids for o in outs0] == [o.token_ids for o in outs] and eng0.stats["prefill_chunks"] == 0
