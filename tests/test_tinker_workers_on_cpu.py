"""Split training primitives: gradient clearing, forward/backward and the optimizer step as separate calls."""

import pytest
import torch

from verl_b200.workers.engine_workers_tinker import OptimStepParams, TinkerActorRolloutRefWorker, _apply_optim_step_params


def _trainer(tmp_path, cls=None):
    from tests.test_trainer_e2e_on_cpu import OV
    from verl_b200.single_controller.base import ClassWithInitArgs
    from verl_b200.single_controller.spmd import SPMDWorkerGroup
    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.utils.config import load_config

    cfg = load_config("ppo_trainer", OV + [f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.total_training_steps=2",
                                           "actor_rollout_ref.actor.optim.lr=1e-3", "actor_rollout_ref.actor.ppo_mini_batch_size=8"])
    tr = PPOTrainer(cfg, reward_fn=load_reward_manager(cfg, None), val_reward_fn=None)
    if cls is not None:
        tr.actor_rollout_wg = SPMDWorkerGroup(cls_with_init_args=ClassWithInitArgs(cls, config=cfg.actor_rollout_ref, role="actor_rollout_ref"))
        tr.ref_policy_wg = tr.actor_rollout_wg
        tr.critic_wg = tr.rm_wg = None
        tr.actor_rollout_wg.init_model()
        tr.actor_rollout_wg.update_weights()
    else:
        tr.init_workers()
    return tr


def test_forward_backward_calls_accumulate_until_the_step(tmp_path):
    ref = _trainer(tmp_path)                                   # plain worker: produces a rollout batch with old log-probs, advantages
    ref.global_steps = 1
    ref.step(next(iter(ref.train_dataloader)))
    batch = ref._last_batch
    n = len(batch)
    halves = (batch[0:n // 2], batch[n // 2:n])

    def run(order):
        tk = _trainer(tmp_path, TinkerActorRolloutRefWorker)
        wg = tk.actor_rollout_wg
        eng = wg.worker.actor.engine
        start = eng.store.flat.clone()
        wg.optimizer_zero_grad()
        outs = [wg.forward_backward(halves[i]) for i in order]
        assert outs[0].batch["log_probs"].shape[0] == n // 2 and "loss" in outs[0].meta_info["metrics"]
        assert torch.equal(eng.store.flat, start)              # nothing moves before the step
        m = wg.optimizer_step()[0]
        assert m["grad_norm"] > 0
        return wg, eng, start, eng.store.flat.clone()

    wg, eng, start, ab = run((0, 1))
    _, _, _, ba = run((1, 0))
    _, _, _, a_only = run((0,))
    assert not torch.equal(ab, start)
    assert torch.allclose(ab, ba, atol=1e-6)                   # accumulation does not depend on the order of the calls
    assert not torch.allclose(ab, a_only, atol=1e-6)           # and the second call did contribute

    # a step-time override applies to that step only
    wg.optimizer_zero_grad()
    wg.forward_backward(halves[0])
    before = eng.store.flat.clone()
    wg.optimizer_step(OptimStepParams(lr=0.0, weight_decay=0.0))
    assert torch.equal(eng.store.flat, before) and eng.lr == pytest.approx(1e-3)


def test_optim_step_params_are_validated():
    class E:
        lr, adam_eps, weight_decay, beta1, beta2 = 1e-3, 1e-8, 0.01, 0.9, 0.999

    e = E()
    saved = _apply_optim_step_params(e, {"lr": 5e-4, "betas": (0.8, 0.9), "eps": None})
    assert (e.lr, e.beta1, e.beta2) == (5e-4, 0.8, 0.9) and saved == {"lr": 1e-3, "beta1": 0.9, "beta2": 0.999}
    with pytest.raises(ValueError):
        _apply_optim_step_params(e, {"momentum": 0.9})
    with pytest.raises(TypeError):
        _apply_optim_step_params(e, {"lr": "fast"})
    with pytest.raises(TypeError):
        _apply_optim_step_params(e, [1, 2])


def test_detach_worker_parks_weights_on_the_host_and_rolls_an_update_back(tmp_path):
    from verl_b200.experimental.separation import DetachActorWorker

    ref = _trainer(tmp_path)
    ref.global_steps = 1
    ref.step(next(iter(ref.train_dataloader)))
    batch = ref._last_batch
    tr = _trainer(tmp_path, DetachActorWorker)
    wg = tr.actor_rollout_wg
    eng = wg.worker.actor.engine
    before_flat, before_master = eng.store.flat.clone(), eng.master.clone()
    assert wg.save_model_to_cpu(0)[0] == before_flat.numel() * before_flat.element_size() + before_master.numel() * 4
    wg.update_actor(batch)
    assert not torch.equal(eng.store.flat, before_flat)
    wg.save_model_to_cpu("after")
    after_flat = eng.store.flat.clone()
    assert wg.restore_model_from_cpu(0) == [True]
    assert torch.equal(eng.store.flat, before_flat) and torch.equal(eng.master, before_master)
    p = next(iter(eng.model.parameters()))
    assert p.data_ptr() >= eng.store.flat.data_ptr()            # parameters are still views of the live buffer
    assert wg.restore_model_from_cpu("after") == [True] and torch.equal(eng.store.flat, after_flat)
    assert wg.saved_model_keys() == [[0, "after"]] and wg.clear_cpu_model(0) == [True] and wg.clear_cpu_model(0) == [False]
    assert wg.restore_model_from_cpu(0) == [False]
