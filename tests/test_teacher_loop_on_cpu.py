"""Served distillation teachers: prompt scoring in the rollout engine / server / HTTP client, routing, padding, fleet layout and one
trainer step against a teacher server process."""

import asyncio

import pytest
import torch

from verl_b200.experimental.teacher_loop import AsyncTeacherLLMServerManager, TeacherModelManager, TeacherModelSpec, build_teacher_fleet, pad_teacher_outputs
from verl_b200.experimental.teacher_loop.teacher_model import check_node_alignment
from verl_b200.models.config import PRESETS
from verl_b200.models.transformer import DecoderLM, PackedBatch
from verl_b200.workers.rollout.async_server import AsyncRolloutServer, serve_http
from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams
from verl_b200.workers.rollout.llm_server import LLMServerClient


def _engine(seed):
    return InferenceEngine(DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=seed), max_num_seqs=8, max_model_len=256, num_blocks=64)


def _oracle(model, seq):
    ids = torch.tensor(seq)
    cu = torch.tensor([0, len(seq)], dtype=torch.int32)
    with torch.no_grad():
        h = model.forward_hidden(PackedBatch(ids, torch.arange(len(seq), dtype=torch.int32), cu, cu, len(seq)))
        return torch.log_softmax(torch.nn.functional.linear(h, model.output_weight).float(), -1)      # row i predicts token i + 1


def test_engine_scores_prompts_topk_and_plain():
    eng = _engine(3)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(10, 2000, (n,), generator=g).tolist() for n in (7, 33, 1, 18)]
    res = eng.score_prompts(seqs, 4, max_tokens_per_pass=40, chunk=16)         # several passes and several vocabulary chunks
    for s, (ids, lps) in zip(seqs, res):
        assert ids.shape == (len(s), 4) and lps.shape == (len(s), 4)
        assert ids[0].tolist() == [s[0]] * 4 and lps[0].abs().sum() == 0
        if len(s) > 1:
            v, ix = _oracle(eng.model, s)[:-1].topk(4, -1)
            assert torch.equal(ids[1:].long(), ix) and torch.allclose(lps[1:], v, atol=1e-5)
    for s, (ids, lps) in zip(seqs, eng.score_prompts(seqs, 0)):
        assert ids[:, 0].tolist() == s
        if len(s) > 1:
            want = _oracle(eng.model, s)[:-1].gather(-1, torch.tensor(s[1:])[:, None]).squeeze(-1)
            assert torch.allclose(lps[1:, 0], want, atol=1e-5)


def test_two_served_teachers_routing_padding_and_http():
    eng_a, eng_b = _engine(5), _engine(6)
    srv_a, srv_b = AsyncRolloutServer(eng_a, name="ta"), AsyncRolloutServer(eng_b, name="tb")
    addr, stop = serve_http(srv_b)                                        # teacher b is reached over HTTP, teacher a in process
    try:
        clients = {"math": LLMServerClient({"ta": srv_a}), "code": LLMServerClient({"tb": addr})}
        with pytest.raises(ValueError, match="do not match teacher routing keys"):
            AsyncTeacherLLMServerManager({"teacher_models": {"math": {}, "qa": {}}}, clients)
        mgr = AsyncTeacherLLMServerManager({"teacher_key": "data_source", "topk": 3, "teacher_models": {"math": {}, "code": {}}}, clients)
        with pytest.raises(ValueError, match="Routing key is required"):
            mgr.resolve_teacher_key(None)
        with pytest.raises(ValueError, match="No teacher configured"):
            mgr.resolve_teacher_key("qa")
        P, R = 6, 5
        prompts = torch.tensor([[0, 0, 11, 12, 13, 14], [21, 22, 23, 24, 25, 26], [0, 0, 0, 0, 31, 32]])
        resp = torch.tensor([[41, 42, 43, 0, 0], [51, 52, 53, 54, 55], [61, 0, 0, 0, 0]])
        att = torch.cat([(prompts != 0).long(), (resp != 0).long()], 1)
        ids, lps = mgr.compute_teacher_topk(prompts, resp, att, ["math", "code", "math"], pad_token_id=0)
        assert ids.shape == (3, R, 3) and lps.shape == (3, R, 3) and ids.dtype == torch.long
        for i, (eng, pl, rl) in enumerate([(eng_a, 4, 3), (eng_b, 6, 5), (eng_a, 2, 1)]):
            seq = prompts[i, P - pl:].tolist() + resp[i, :rl].tolist()
            v, ix = _oracle(eng.model, seq)[pl - 1:pl - 1 + rl].topk(3, -1)      # the prediction for response token j is made at row pl - 1 + j
            assert torch.equal(ids[i, :rl], ix) and torch.allclose(lps[i, :rl], v, atol=1e-4)
            assert ids[i, rl:].abs().sum() == 0 and lps[i, rl:].abs().sum() == 0
        # a generation request on the same server still works and is not mixed into the scoring batch
        out = asyncio.run(clients["math"].generate("g", [5, 6, 7], SamplingParams(temperature=0.0, max_tokens=3)))
        assert len(out.token_ids) == 3 and not out.extra_fields
        a, b = pad_teacher_outputs(torch.ones(4, 2, dtype=torch.int32), torch.ones(4, 2), 5, 3, 3, 1, 9)
        assert a.shape == (1, 8, 2) and a[0, :2].eq(9).all() and a[0, 6:].eq(9).all() and b[0, :2].eq(0).all()
        with pytest.raises(ValueError, match="rows for a sequence"):
            pad_teacher_outputs(torch.ones(4, 2), torch.ones(4, 2), 5, 3, 2, 1, 0)
        asyncio.run(clients["code"].close())
    finally:
        stop()
        srv_a.shutdown()
        srv_b.shutdown()


def test_fleet_layout_checks():
    check_node_alignment("a", 0, 2, 4, 8)
    check_node_alignment("wide", 0, 1, 16, 8)
    with pytest.raises(ValueError, match="span 2 node"):
        check_node_alignment("b", 3, 1, 4, 4)                                # devices [3, 7) of 4-GPU nodes straddle two nodes
    spec = TeacherModelSpec.from_config("math", {"model_path": "tiny-qwen2", "num_replicas": 2, "inference": {"max_model_len": 128}})
    assert spec.per_replica_world_size == 1 and spec.max_model_len == 128
    with pytest.raises(ValueError, match="expected 2 devices"):
        TeacherModelManager(spec, ["0"])
    with pytest.raises(ValueError, match="need 3 devices"):
        build_teacher_fleet({"a": {"model_path": "x", "num_replicas": 2}, "b": {"model_path": "y"}}, ["0", "1"])
    with pytest.raises(ValueError, match="model_path is required"):
        TeacherModelSpec.from_config("c", {})
    m = TeacherModelManager(spec, [], servers={"s0": "127.0.0.1:1"})
    assert m.prometheus_targets() == ["127.0.0.1:1"] and isinstance(m.client(), LLMServerClient)


def test_trainer_step_distils_from_a_teacher_server_process(tmp_path):
    """``distillation.teacher_mode=server``: the trainer starts the teacher fleet (one standalone server process), fetches the
    teacher's top-k head for every sample through it and the actor minimises the forward KL to it; no colocated teacher exists."""
    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.utils.config import load_config

    ov = ["data.synthetic.enable=true", "data.synthetic.num_prompts=64", "data.train_batch_size=4", "data.max_prompt_length=32",
          "data.max_response_length=8", "actor_rollout_ref.model.preset=tiny-qwen2", "actor_rollout_ref.rollout.n=2",
          "actor_rollout_ref.actor.ppo_mini_batch_size=2", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
          "actor_rollout_ref.actor.use_kl_loss=false", "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8",
          "actor_rollout_ref.rollout.max_num_seqs=8", "actor_rollout_ref.model.enable_gradient_checkpointing=false",
          "actor_rollout_ref.actor.optim.lr=3e-3", "actor_rollout_ref.distillation.enable=true", "actor_rollout_ref.distillation.teacher_mode=server",
          "actor_rollout_ref.distillation.teacher_model.preset=tiny-qwen2", "actor_rollout_ref.distillation.topk=8",
          "+actor_rollout_ref.actor.fsdp_config.seed=1", "algorithm.adv_estimator=grpo", "reward.reward_manager=token_rule", "trainer.device=cpu",
          "trainer.val_before_train=false", "trainer.logger=[]", "trainer.n_gpus_per_node=1", "data.shuffle=false",
          f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.total_training_steps=2"]
    cfg = load_config("ppo_trainer", ov)
    tr = PPOTrainer(cfg, reward_fn=load_reward_manager(cfg, None), val_reward_fn=None)
    tr.init_workers()
    assert tr.actor_rollout_wg.worker.teacher is None
    try:
        it = iter(tr.train_dataloader)
        for step in (1, 2):
            tr.global_steps = step
            m = tr.step(next(it))
            assert "timing_s/teacher" in m and m["distill/forward_kl"] > 0 and 0.0 <= m["distill/top1_agreement"] <= 1.0
        b = tr._last_batch.batch
        assert b["teacher_topk_ids"].shape == (8, 8, 8) and (b["teacher_topk_log_probs"][..., 0] >= b["teacher_topk_log_probs"][..., 1]).all()
        fleet = tr._teacher_fleet["default"]
        assert len(fleet.rollout_replicas) == 1 and fleet.rollout_replicas[0]._proc.poll() is None
    finally:
        for f in getattr(tr, "_teacher_fleet", {}).values():
            f.shutdown()
