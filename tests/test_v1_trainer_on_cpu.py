"""TransferQueue, replay buffers and the v1 trainers (sync and colocated-async) on the CPU plumbing configuration."""

import json

import torch

from tests.test_trainer_e2e_on_cpu import OV
from verl_b200.protocol import DataProto
from verl_b200.trainer.ppo.reward import load_reward_manager
from verl_b200.trainer.ppo.v1 import ReplayBuffer, ReplayBufferAsync, get_trainer_cls
from verl_b200.trainer.ppo.v1.checkpoint_callback import CheckpointCallback
from verl_b200.utils.config import load_config
from verl_b200.utils.transfer_queue import KVBatchMeta, TransferQueue, tqbridge


def test_transfer_queue_roundtrip_and_bridge():
    tq = TransferQueue()
    data = DataProto.from_dict(tensors={"x": torch.arange(6).reshape(3, 2)}, non_tensors={"name": ["a", "b", "c"]})
    meta = KVBatchMeta("p", ["k0", "k1", "k2"])
    tq.kv_batch_put(meta, data, tags={"status": "finished"})
    got = tq.kv_get(KVBatchMeta("p", ["k2", "k0"], ["x", "name"]))
    assert got.batch["x"].tolist() == [[4, 5], [0, 1]] and got.non_tensor_batch["name"].tolist() == ["c", "a"]
    assert tq.kv_tags("p")["k1"]["status"] == "finished" and tq.size("p") == 3

    import verl_b200.utils.transfer_queue as mod

    mod._TQ = tq

    class W:
        @tqbridge()
        def double(self, d: DataProto) -> DataProto:
            return DataProto.from_dict(tensors={"y": d.batch["x"] * 2})

    m2 = W().double(KVBatchMeta("p", ["k0", "k1"], ["x"]))
    assert isinstance(m2, KVBatchMeta) and "y" in m2.fields
    assert tq.kv_get(KVBatchMeta("p", ["k1"], ["y"])).batch["y"].tolist() == [[4, 6]]
    assert W().double(data).batch["y"].shape == (3, 2)       # plain batches pass through
    mod._TQ = None


def test_replay_buffer_groups_filters_and_staleness():
    tq = TransferQueue()
    for uid, scores, step, status in (("a", (1.0, 0.0), 1, "finished"), ("b", (1.0, 1.0), 1, "finished"), ("c", (0.0, 1.0), 3, "finished"),
                                      ("d", (0.0, 1.0), 3, "running"), ("e", (0.0, 1.0), 3, "failure")):
        for j, sc in enumerate(scores):
            tq.kv_put("train", f"{uid}#{j}", {"v": torch.tensor(j)}, {"uid": uid, "status": status if j else "finished", "gen_step": step, "score": sc})
    rb = ReplayBuffer(tq, rollout_n=2, filter_groups=True)
    assert rb.get_sampleable_count(3, "train") == 2            # b filtered (equal scores), d running, e failed
    meta, m = rb.sample(3, "train", 2)
    assert meta.keys == ["a#0", "a#1", "c#0", "c#1"] and m["replay/evicted_filtered"] == 1 and m["replay/evicted_failure"] == 1
    assert "b#0" not in tq.kv_tags("train") and "d#0" in tq.kv_tags("train")
    rba = ReplayBufferAsync(tq, rollout_n=2, max_off_policy_threshold=1)
    assert rba.get_sampleable_count(3, "train") == 1           # group a (step 1) is two steps old at step 3
    cb = CheckpointCallback({"save_freq": 2})
    assert [cb.should_save(i, False) for i in (1, 2, 3)] == [False, True, False] and cb.should_save(3, True)


def _run(tmp_path, name, extra=()):
    logf = tmp_path / f"{name}.jsonl"
    import os

    os.environ["VERL_FILE_LOGGER_PATH"] = str(logf)
    try:
        cfg = load_config("ppo_trainer", [o for o in OV if not o.startswith("trainer.logger")] +
                          ["trainer.logger=[file]", "trainer.total_training_steps=3", f"trainer.default_local_dir={tmp_path}/ckpt_{name}",
                           "actor_rollout_ref.rollout.mode=async", "actor_rollout_ref.rollout.free_cache_engine=false",
                           "trainer.resume_mode=disable"] + list(extra))
        tr = get_trainer_cls(name)(cfg, reward_fn=load_reward_manager(cfg, None))
        tr.init()
        tr.fit()
    finally:
        os.environ.pop("VERL_FILE_LOGGER_PATH", None)
    return [json.loads(x)["data"] for x in logf.read_text().splitlines()]


def test_v1_sync_trainer_is_on_policy(tmp_path):
    rows = _run(tmp_path, "sync")
    assert len(rows) == 3 and all(r["replay/staleness_max"] == 0 for r in rows) and rows[-1]["perf/total_num_tokens"] > 0
    assert abs(rows[0]["actor/ppo_kl"]) < 1e-4


def test_v1_colocate_async_trainer_runs_ahead(tmp_path):
    rows = _run(tmp_path, "colocate_async", ["+trainer.v1.async_warmup_batches=1", "+trainer.v1.max_off_policy_threshold=2"])
    assert len(rows) == 3 and max(r["replay/staleness_max"] for r in rows) >= 1 and rows[-1]["perf/total_num_tokens"] > 0


def test_one_step_off_policy_and_fully_async_trainers(tmp_path):
    import verl_b200.experimental.fully_async_policy  # noqa: F401 - registers "fully_async"
    import verl_b200.experimental.one_step_off_policy  # noqa: F401 - registers "one_step_off_policy"

    rows = _run(tmp_path, "one_step_off_policy")
    assert len(rows) == 3 and [r["replay/staleness_max"] for r in rows] == [1, 1, 1]
    rows = _run(tmp_path, "fully_async", ["+trainer.v1.staleness_threshold=3", "+trainer.v1.queue_batches=2"])
    assert len(rows) == 3 and rows[-1]["perf/total_num_tokens"] > 0 and max(r["replay/staleness_max"] for r in rows) <= 3


def test_distillation_losses():
    from verl_b200.trainer.distillation import forward_kl, jsd, reverse_kl, topk_distillation_loss

    torch.manual_seed(0)
    t = torch.log_softmax(torch.randn(6, 30), -1)
    s = torch.log_softmax(torch.randn(6, 30), -1).requires_grad_(True)
    idx = t.topk(5).indices
    th, sh = t.gather(-1, idx), s.gather(-1, idx)
    for f in (forward_kl, reverse_kl, jsd):
        assert (f(sh, th) >= -1e-6).all() and f(th, th).abs().max() < 1e-6
    # with the whole vocabulary in the head the forward KL is the exact KL
    full = forward_kl(s, t)
    assert torch.allclose(full, (t.exp() * (t - s)).sum(-1), atol=1e-4)
    loss, m = topk_distillation_loss(sh, th, torch.ones(2, 3), "jsd")
    loss.backward()
    assert s.grad is not None and 0 <= m["distill/top1_agreement"] <= 1


def test_v1_separate_async_trainer_feeds_a_standalone_replica_and_pushes_weights(tmp_path):
    """Rollout runs in its own server process; the trainer streams prompts to it over HTTP and hands over new weights after
    every update (file hand-off on CPU). The replica ends with exactly the trainer's weights."""
    import os

    logf = tmp_path / "sep.jsonl"
    os.environ["VERL_FILE_LOGGER_PATH"] = str(logf)
    try:
        cfg = load_config("ppo_trainer", [o for o in OV if not o.startswith("trainer.logger")] +
                          ["trainer.logger=[file]", "trainer.total_training_steps=2", f"trainer.default_local_dir={tmp_path}/ckpt_sep",
                           "actor_rollout_ref.rollout.mode=async", "actor_rollout_ref.rollout.free_cache_engine=false", "trainer.resume_mode=disable",
                           "+trainer.v1.max_off_policy_threshold=3", "+trainer.v1.async_warmup_batches=1", "+trainer.v1.rollout_num_blocks=64"])
        tr = get_trainer_cls("separate_async")(cfg, reward_fn=load_reward_manager(cfg, None))
        tr.init()
        assert len(tr.replicas) == 1 and tr.replicas[0].address and tr.replicas[0]._proc is not None
        replica = tr.replicas[0]
        orig_end = tr.on_train_end
        seen = {}

        def end():
            seen.update(replica.weights_version(checksum=True))
            orig_end()

        tr.on_train_end = end
        tr.fit()
    finally:
        os.environ.pop("VERL_FILE_LOGGER_PATH", None)
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 2 and rows[-1]["sync/param_version"] == 3 and rows[-1]["perf/total_num_tokens"] > 0
    assert seen["weights_version"] == 3                       # initial hand-off + one per step
    eng = tr.stages.actor_rollout_wg.worker.actor.engine
    want = float(sum(p.detach().double().sum() for p in eng.model.parameters()))
    assert abs(seen["checksum"] - want) < 1e-6 * max(1.0, abs(want))
    assert replica._proc.poll() is not None                   # the pool was shut down with the trainer


def test_v1_separate_async_lends_the_training_engine_while_it_would_wait(tmp_path):
    """Hybrid lending: after a step the colocated engine joins the balancer and serves requests until the switch threshold of
    the next batch is sampleable; then it is taken back (its open requests move to the pool) and training proceeds. The
    threshold adapts and the decision metrics are logged."""
    import os

    from verl_b200.trainer.ppo.v1.trainer_separate_async import HybridEngineMode

    logf = tmp_path / "lend.jsonl"
    os.environ["VERL_FILE_LOGGER_PATH"] = str(logf)
    try:
        cfg = load_config("ppo_trainer", [o for o in OV if not o.startswith("trainer.logger")] +
                          ["trainer.logger=[file]", "trainer.total_training_steps=3", f"trainer.default_local_dir={tmp_path}/ckpt_lend",
                           "actor_rollout_ref.rollout.mode=async", "actor_rollout_ref.rollout.free_cache_engine=false", "trainer.resume_mode=disable",
                           "+trainer.v1.max_off_policy_threshold=4", "+trainer.v1.async_warmup_batches=0", "+trainer.v1.rollout_num_blocks=64",
                           "trainer.v1.separate_async.hybrid_rollout.enable_switch=true", "trainer.v1.separate_async.hybrid_rollout.switch_threshold_ratio=0.5"])
        tr = get_trainer_cls("separate_async")(cfg, reward_fn=load_reward_manager(cfg, None))
        tr.init()
        assert tr._switch_enabled and tr.current_mode == HybridEngineMode.TRAINER
        assert tr._switch_threshold() == max(1, round(0.5 * tr.train_batch_size))
        served_before = tr._hybrid_replica.server.stats.get("finished", 0)
        tr.fit()
    finally:
        os.environ.pop("VERL_FILE_LOGGER_PATH", None)
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 3 and all(r["perf/total_num_tokens"] > 0 for r in rows)
    # with no warm-up batch every step waits for its trajectories: the trainer lent its engine after steps 1 and 2 ...
    kinds = [k for k, _ in tr.switch_log]
    assert kinds.count("rollout") >= 1 and kinds.count("trainer") == kinds.count("rollout")
    assert tr.current_mode == HybridEngineMode.TRAINER
    assert rows[0]["separate_async/decision/should_switch_to_rollout"] == 1.0 and rows[-1]["separate_async/decision/should_switch_to_rollout"] == 0.0
    assert "separate_async/switch/threshold_ratio" in rows[0] and rows[0]["separate_async/switch/idle"] == 1.0
    # ... and the lent engine really served requests
    assert tr._hybrid_replica.server.stats.get("finished", 0) + tr._hybrid_replica.server.stats.get("aborted", 0) > served_before
    # adaptive threshold: repeated idle steps push the ratio up, calm ones bring it down to one mini-batch at the lowest
    tr._switch_threshold_ratio, tr._idle_steps, tr._calm_steps = 0.5, 0, 0
    for _ in range(2):
        tr._adapt_switch_threshold(True)
    assert abs(tr._switch_threshold_ratio - 0.55) < 1e-9
    for _ in range(40):
        tr._adapt_switch_threshold(False)
    assert abs(tr._switch_threshold_ratio - 1.0 / tr.parameter_sync_step) < 1e-9


def test_v1_separate_async_lending_driven_by_a_registered_policy(tmp_path):
    """The same lending, decided by a pluggable dynamic-schedule policy (``hybrid_rollout.policy``) through the resource
    controller: the fixed-ratio policy lends after every step that leaves a gap and takes the engine back at ratio x batch."""
    import os

    from verl_b200.experimental.fully_async_policy.dynamic_schedule import FixedRatioDynamicSchedulePolicy
    from verl_b200.trainer.ppo.v1.trainer_separate_async import HybridEngineMode

    logf = tmp_path / "lend_policy.jsonl"
    os.environ["VERL_FILE_LOGGER_PATH"] = str(logf)
    try:
        cfg = load_config("ppo_trainer", [o for o in OV if not o.startswith("trainer.logger")] +
                          ["trainer.logger=[file]", "trainer.total_training_steps=3", f"trainer.default_local_dir={tmp_path}/ckpt_lend_policy",
                           "actor_rollout_ref.rollout.mode=async", "actor_rollout_ref.rollout.free_cache_engine=false", "trainer.resume_mode=disable",
                           "+trainer.v1.max_off_policy_threshold=4", "+trainer.v1.async_warmup_batches=0", "+trainer.v1.rollout_num_blocks=64",
                           "trainer.v1.separate_async.hybrid_rollout.enable_switch=true", "trainer.v1.separate_async.hybrid_rollout.switch_threshold_ratio=0.5",
                           "trainer.v1.separate_async.hybrid_rollout.policy=fixed_ratio"])
        tr = get_trainer_cls("separate_async")(cfg, reward_fn=load_reward_manager(cfg, None))
        tr.init()
        ctl = tr._controller
        assert isinstance(ctl.policy, FixedRatioDynamicSchedulePolicy) and ctl.policy.deactivate_ratio == 0.5 and not ctl.only_hybrid
        assert tr._switch_threshold() == tr.train_batch_size            # nothing lent yet: the policy asks for no take-back
        tr.fit()
    finally:
        os.environ.pop("VERL_FILE_LOGGER_PATH", None)
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 3 and all(r["perf/total_num_tokens"] > 0 for r in rows)
    assert ctl.activate_count >= 1 and ctl.activate_count == ctl.deactivate_count and not ctl.is_hybrid_active
    assert [k for k, _ in tr.switch_log].count("rollout") == ctl.activate_count and tr.current_mode == HybridEngineMode.TRAINER
    assert rows[0]["dynamic_schedule/want_activate"] == 1.0 and rows[-1]["dynamic_schedule/want_activate"] == 0.0    # no step left to lend for
    assert rows[0]["dynamic_schedule/deactivate_ratio"] == 0.5 and ctl.last_activate_duration_s > 0 and ctl.last_deactivate_duration_s > 0


def test_transfer_queue_over_tcp_between_processes(tmp_path):
    """A served TransferQueue: a child process writes trajectories, this process blocks on the server until they are tagged
    finished, reads them back as a batch and sees the child's tags; server-side errors come back as exceptions."""
    import subprocess
    import sys

    import pytest

    from verl_b200.utils.transfer_queue_remote import RemoteTransferQueue, TransferQueueServer

    srv = TransferQueueServer()
    child = (
        "import sys, torch\n"
        "from verl_b200.protocol import DataProto\n"
        "from verl_b200.utils.transfer_queue import KVBatchMeta\n"
        "from verl_b200.utils.transfer_queue_remote import RemoteTransferQueue\n"
        "q = RemoteTransferQueue(sys.argv[1])\n"
        "d = DataProto.from_dict(tensors={'x': torch.arange(8).reshape(4, 2)}, non_tensors={'name': ['a', 'b', 'c', 'd']})\n"
        "q.kv_batch_put(KVBatchMeta('train', ['k0', 'k1', 'k2', 'k3']), d, tags={'status': 'finished', 'gen_step': 3})\n"
        "q.kv_put('train', 'k4', tags={'status': 'running'})\n"
    )
    import os

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.Popen([sys.executable, "-c", child, srv.address], env=dict(os.environ, PYTHONPATH=repo))
    q = RemoteTransferQueue(srv.address)
    try:
        assert q.wait_for_tags("train", 4, {"status": "finished"}, timeout=120)
        assert p.wait(timeout=60) == 0
        got = q.kv_get(KVBatchMeta("train", ["k2", "k0"], ["x", "name"]))
        assert got.batch["x"].tolist() == [[4, 5], [0, 1]] and got.non_tensor_batch["name"].tolist() == ["c", "a"]
        tags = q.kv_tags("train")
        assert tags["k1"] == {"status": "finished", "gen_step": 3} and tags["k4"]["status"] == "running" and q.size("train") == 5
        assert not q.wait_for_tags("train", 5, {"status": "finished"}, timeout=0.2)
        q.kv_clear("train", ["k4"])
        assert srv.queue.size("train") == 4                     # the server's store is the one being edited
        with pytest.raises(RuntimeError, match="KeyError"):
            q.kv_get(KVBatchMeta("train", ["missing"]))
        rb = ReplayBuffer(q, rollout_n=1)                       # the replay buffer works against the remote store unchanged
        assert rb.get_sampleable_count(3, "train") == 4
    finally:
        q.close()
        srv.shutdown()
