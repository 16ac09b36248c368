"""Headline benchmark: GRPO step throughput (rollout + log-prob passes + actor update + weight hand-off) on the
Qwen2.5-7B architecture, one process per GPU.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 2 --warmup 3

Weak scaling: every GPU owns 32 prompts x n=8 samples per step (256 prompts x 8 on 8 GPUs, the configuration the
baseline names), PPO mini-batch 8 prompts per GPU (64 on 8 GPUs). Synthetic prompts (lengths uniform in [256, 512],
ids uniform in [100, 150000)), random-init weights, response length up to 1024, temperature 1.0, clip 0.2,
low-variance KL loss 1e-3 against a frozen reference, packed (remove-padding) batches with a token budget per
micro-batch. ``value`` is tokens (prompt + response, whole job) per second over the timed steps, timed with CUDA
events and taken as the max over ranks; ``e2e`` is the same metric from wall clock around the public
``PPOTrainer.step`` call including the data-loader fetch, pinned host-to-device input copies and the device-to-host
read of every result.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

# The reference publishes no number for this configuration and its package cannot be installed offline (no ray / tensordict /
# hydra wheels), so the anchor is the same GRPO step built from the stock libraries the reference
# calls (vLLM 0.22 rollout, transformers + FlashAttention-2 + torch AdamW training; `--impl stocklibs`), measured on one B200:
# 6528 tokens/s per GPU. vs_baseline = value / (n_gpus x that number), i.e. the baseline is granted perfect weak scaling.
BASELINE_PUBLISHED = 6528.2


def _job_start_time() -> float:
    """Wall-clock time at which this job began: the launcher's start when run under ``torch.distributed.run`` (its own
    ``import torch`` on a cold machine can take a minute before any rank exists), else this process's."""
    t = time.time()
    try:
        import psutil

        me = psutil.Process()
        t = min(t, me.create_time())
        parent = me.parent()
        if parent is not None and any("torch.distributed.run" in a or a.endswith("torchrun") for a in parent.cmdline()):
            t = min(t, parent.create_time())
    except Exception:  # noqa: BLE001
        pass
    return t


T_PROCESS_START = _job_start_time()
MIN_WARMUP = 3          # never time a step before three warm-up steps have run


def _clock_sampler(stop: threading.Event, out: list, gpu_index: int):
    q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    while not stop.is_set():
        try:
            r = subprocess.run(["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                               capture_output=True, text=True, timeout=5)
            if r.returncode == 0 and r.stdout.strip():
                out.append([x.strip() for x in r.stdout.strip().splitlines()[0].split(",")])
        except Exception:  # noqa: BLE001
            pass
        stop.wait(0.2)


def _summarise_clocks(samples: list) -> dict:
    if not samples:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
    sm = sorted(float(s[0]) for s in samples if s[0].replace(".", "").isdigit())
    mx = max((float(s[1]) for s in samples if s[1].replace(".", "").isdigit()), default=None)
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    reasons = [n for i, n in enumerate(names) if any(len(s) > 3 + i and s[3 + i].lower().startswith("active") for s in samples)]
    return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons, "samples": len(samples)}


def build_config(args, world: int):
    from verl_b200.utils.config import load_config

    prompts_per_gpu = args.prompts_per_gpu
    ov = [
        "data.synthetic.enable=true", f"data.synthetic.num_prompts={prompts_per_gpu * world * (args.steps + args.warmup + 1)}",
        f"data.synthetic.min_prompt_length={args.min_prompt}", f"data.synthetic.max_prompt_length={args.max_prompt}",
        "data.synthetic.id_low=100", "data.synthetic.id_high=150000",
        f"data.train_batch_size={prompts_per_gpu * world}", f"data.max_prompt_length={args.max_prompt}",
        f"data.max_response_length={args.response_length}", "data.shuffle=false", "data.seed=0",
        f"actor_rollout_ref.model.preset={args.model}", "actor_rollout_ref.model.enable_gradient_checkpointing=" + ("true" if args.grad_ckpt else "false"),
        f"actor_rollout_ref.rollout.n={args.n}", "actor_rollout_ref.rollout.temperature=1.0", "actor_rollout_ref.rollout.ignore_eos=false",
        f"actor_rollout_ref.rollout.max_num_seqs={prompts_per_gpu * args.n}", f"actor_rollout_ref.rollout.gpu_memory_utilization={args.kv_util}",
        f"actor_rollout_ref.actor.ppo_mini_batch_size={args.mini_prompts_per_gpu * world}",
        "actor_rollout_ref.actor.use_dynamic_bsz=true", f"actor_rollout_ref.actor.ppo_max_token_len_per_gpu={args.token_budget}",
        "actor_rollout_ref.rollout.log_prob_use_dynamic_bsz=true", f"actor_rollout_ref.rollout.log_prob_max_token_len_per_gpu={args.token_budget * 2}",
        "actor_rollout_ref.ref.log_prob_use_dynamic_bsz=true", f"actor_rollout_ref.ref.log_prob_max_token_len_per_gpu={args.token_budget * 2}",
        "actor_rollout_ref.actor.use_kl_loss=true", "actor_rollout_ref.actor.kl_loss_coef=0.001", "actor_rollout_ref.actor.kl_loss_type=low_var_kl",
        "actor_rollout_ref.actor.clip_ratio=0.2", "algorithm.adv_estimator=grpo", "reward.reward_manager=token_rule",
        "trainer.val_before_train=false", "trainer.balance_batch=true", "trainer.logger=[]", "trainer.worker_backend=spmd",
        f"trainer.n_gpus_per_node={world}", "trainer.nnodes=1", f"trainer.total_training_steps={args.steps + args.warmup}",
        "trainer.resume_mode=disable", "trainer.save_freq=-1",
    ]
    if args.ref_offload:
        ov.append("actor_rollout_ref.ref.fsdp_config.param_offload=true")
    if args.prefix_sharing:
        ov.append("actor_rollout_ref.actor.use_prefix_grouper=true")
    if args.rollout_quant:
        ov.append(f"actor_rollout_ref.rollout.quantization={args.rollout_quant}")
    if args.zero3:
        ov += ["actor_rollout_ref.actor.fsdp_config.reshard_after_forward=true", "+actor_rollout_ref.ref.fsdp_config.reshard_after_forward=true"]
    if args.rollout_tp > 1:
        ov.append(f"actor_rollout_ref.rollout.tensor_model_parallel_size={args.rollout_tp}")
        ov.append(f"actor_rollout_ref.rollout.max_num_seqs={prompts_per_gpu * args.n * args.rollout_tp}")
    return load_config("ppo_trainer", ov)


def run_native(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun --nproc-per-node {args.gpus}"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    from verl_b200.ops import _ext
    from verl_b200.single_controller.spmd import init_spmd_process_group
    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.workers.engine.fsdp.engine import IO_STATS

    _ext.load()
    init_spmd_process_group()
    cfg = build_config(args, world)
    reward_fn = load_reward_manager(cfg, None)
    trainer = PPOTrainer(cfg, tokenizer=None, reward_fn=reward_fn, val_reward_fn=None)
    trainer.init_workers()
    it = iter(trainer.train_dataloader)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def agree(x: float, op) -> float:
        """One number every rank agrees on (decisions about how many steps to run must not diverge between ranks)."""
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=op)
        return float(t.item())

    def elapsed() -> float:
        return agree(time.time() - T_PROCESS_START, dist.ReduceOp.MAX)

    # Wall-clock guard. A step of this benchmark takes tens of seconds, so `--steps 20 --warmup 5` can exceed the time a
    # caller allows per run. The guard keeps at least three warm-up steps (CUDA-graph capture, allocator steady state),
    # then runs as many timed steps as fit below --time-limit seconds of process wall clock, and reports what it ran.
    limit = float(args.time_limit)
    trainer.global_steps = 1
    warm_times: list = []
    warm_done = 0
    for w in range(args.warmup):
        if limit > 0 and warm_done >= MIN_WARMUP:
            est = max(warm_times[1:] or warm_times)
            if elapsed() + est * (args.warmup - warm_done + max(1, args.steps)) > limit:
                break                           # the remaining warm-up steps would eat the timed steps
        t0 = time.perf_counter()
        m = trainer.step(next(it))
        torch.cuda.synchronize()
        warm_times.append(agree(time.perf_counter() - t0, dist.ReduceOp.MAX))
        warm_done += 1
        trainer.global_steps += 1
        if rank == 0 and args.verbose:
            print(f"[warmup {w}] " + " ".join(f"{k}={v:.3f}" for k, v in m.items() if k.startswith("timing_s/") or k in ("perf/throughput", "actor/grad_norm")), file=sys.stderr, flush=True)
    _ext.check_status("bench warm-up")
    steps_planned = args.steps
    if limit > 0 and warm_times:
        est = max(warm_times[1:] or warm_times) * 1.03
        fit = int((limit - elapsed()) // est)
        steps_planned = max(1, min(args.steps, fit))
    samples: list = []
    stop = threading.Event()
    th = threading.Thread(target=_clock_sampler, args=(stop, samples, local_rank), daemon=True)
    barrier()
    launches0 = _ext.launch_count()
    io0 = dict(IO_STATS)
    th.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    ev0.record()
    tokens = 0
    per_step: list = []
    steps_run = 0
    for s in range(steps_planned):
        batch = next(it)                     # data-loader fetch is part of the end-to-end region
        last = trainer.step(batch)
        trainer.global_steps += 1
        steps_run += 1
        tokens += int(last["perf/total_num_tokens"])
        per_step.append({k.split("/", 1)[1]: round(v, 3) for k, v in last.items() if k.startswith("timing_s/")})
        if rank == 0 and args.verbose:
            print(f"[step {s}] " + " ".join(f"{k}={v:.3f}" for k, v in last.items() if k.startswith("timing_s/") or k in ("perf/throughput", "actor/grad_norm")), file=sys.stderr, flush=True)
        if limit > 0 and s + 1 < steps_planned:
            # safety net for a step that ran much longer than the warm-up steps suggested (one 8-byte all-reduce per step)
            # (the ranks must take the same decision: the projected finish time is agreed as the max over ranks)
            if agree(time.time() - T_PROCESS_START + per_step[-1].get("step", 0.0) * 1.03, dist.ReduceOp.MAX) > limit + 30.0:
                break
    ev1.record()
    barrier()
    t_wall = time.perf_counter() - t_wall0
    stop.set()
    th.join(timeout=2)
    dev_ms = ev0.elapsed_time(ev1)
    launches = _ext.launch_count() - launches0
    _ext.check_status("bench timed region")
    t = torch.tensor([dev_ms, t_wall * 1000.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = t.tolist()
    if rank == 0:
        value = tokens / (dev_ms / 1000.0)
        e2e = tokens / (wall_ms / 1000.0)
        h2d = (IO_STATS["h2d_bytes"] - io0["h2d_bytes"]) / steps_run
        d2h = (IO_STATS["d2h_bytes"] - io0["d2h_bytes"]) / steps_run
        keys = sorted({k for d in per_step for k in d})
        out = {
            "metric": "GRPO step tokens/s (rollout+train), Qwen2.5-7B arch", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": steps_run, "warmup": warm_done, "steps_requested": args.steps, "warmup_requested": args.warmup,
            "ms_per_step": dev_ms / steps_run, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / (BASELINE_PUBLISHED * world)) if BASELINE_PUBLISHED else None, "dtype": "bf16" if not args.rollout_quant else f"bf16 training, {args.rollout_quant} rollout projections", "data": "synthetic prompts, random-init weights",
            "impl": "native",
            "config": {"model": args.model, "global_batch": f"{args.prompts_per_gpu * world} prompts x n={args.n}",
                       "seq_len": f"prompt U[{args.min_prompt},{args.max_prompt}] + response <= {args.response_length}",
                       "parallelism": f"dp{world} ({'ZeRO-3 row-sharded projections gathered inside the GEMMs' if args.zero3 else 'ZeRO-2 sharded optimizer, resident bf16 params'}), rollout tp{args.rollout_tp} x {world // args.rollout_tp} replicas colocated",
                       "ppo_mini_batch_prompts": args.mini_prompts_per_gpu * world, "token_budget_per_micro_batch": args.token_budget,
                       "gradient_checkpointing": bool(args.grad_ckpt), "ref_param_offload": bool(args.ref_offload), "prefix_sharing": bool(args.prefix_sharing), "rollout_quantization": args.rollout_quant or None, "zero3": bool(args.zero3), "loss": "grpo clip 0.2 + low_var_kl 1e-3, AdamW lr 1e-6",
                       "l2_policy": "inputs larger than L2: each step streams >15 GB of weights and fresh activations",
                       "time_limit_s": limit if limit > 0 else None},
            "clocks": _summarise_clocks(samples),
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "step_breakdown_s": {k: [d.get(k) for d in per_step] for k in keys},
            "warmup_step_s": [round(x, 3) for x in warm_times],
            "tokens_per_step": tokens / steps_run,
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 1),
            "native_fallbacks": dict(__import__("verl_b200.ops.functional", fromlist=["fallback_counts"]).fallback_counts),
            # allocator pressure on rank 0: a retry means cudaMalloc failed once and cached blocks were freed (a device sync)
            "allocator": {"reserved_gb": round(torch.cuda.max_memory_reserved() / 1e9, 1),
                          "alloc_retries": int(torch.cuda.memory_stats().get("num_alloc_retries", 0)),
                          "ooms": int(torch.cuda.memory_stats().get("num_ooms", 0))},
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """Runs the unmodified reference installed under ``baseline/_ref`` through its own entry point — if it can start.
    Its package imports ray / tensordict / hydra / omegaconf at import time (``verl/protocol.py``, ``verl/trainer/main_ppo.py``);
    where those are not installed the arm reports itself unavailable instead of substituting anything of ours."""
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref_dir, "verl")):
        why = "reference is not installed under baseline/_ref"
    else:
        sys.path.insert(0, ref_dir)
        try:
            import importlib

            importlib.import_module("verl.trainer.main_ppo")
            why = ("reference imports, but its stock GRPO path needs a Ray cluster, a vLLM/SGLang rollout server and an HF checkpoint + "
                   "parquet dataset on disk; none can be provided offline, so no like-for-like run is possible")
        except Exception as e:  # noqa: BLE001
            why = f"reference entry point cannot be imported offline: {type(e).__name__}: {e}"
        finally:
            sys.path.remove(ref_dir)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "stocklibs"],
                    help="native: this framework; reference: the unmodified reference package under baseline/_ref; stocklibs: the same GRPO "
                         "step from vLLM + transformers/FlashAttention-2 + torch AdamW only (benchmarks/stocklibs_grpo.py, one GPU)")
    ap.add_argument("--vllm-util", type=float, default=0.25, help="stocklibs arm: vLLM gpu_memory_utilization (weights 15 GB + KV cache for 256 x 1536 tokens = 23 GB fit in 0.25 x 180 GB)")
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=32)
    ap.add_argument("--mini-prompts-per-gpu", type=int, default=8)
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--min-prompt", type=int, default=256)
    ap.add_argument("--max-prompt", type=int, default=512)
    ap.add_argument("--response-length", type=int, default=1024)
    ap.add_argument("--token-budget", type=int, default=0, help="tokens per training micro-batch; 0 = 16384 with recomputation, 8192 without")
    ap.add_argument("--kv-util", type=float, default=0.3)
    ap.add_argument("--grad-ckpt", type=int, default=-1,
                    help="activation recomputation (default off: activations of an 8192-token micro-batch are stored)")
    ap.add_argument("--rollout-quant", type=str, default="", help="fp8: W8A8 rollout projections (not the headline config; dtype is then reported as bf16+fp8 rollout)")
    ap.add_argument("--zero3", type=int, default=0, help="row-shard the actor's and the reference's decoder projections over all ranks (weight gather fused into the GEMMs)")
    ap.add_argument("--prefix-sharing", type=int, default=0,
                    help="forward/backward every distinct prompt once for its n responses (actor.use_prefix_grouper); off = the reference's default")
    ap.add_argument("--ref-offload", type=int, default=-1, help="keep the frozen reference weights in pinned host memory between its passes")
    ap.add_argument("--rollout-tp", type=int, default=0,
                    help="GPUs per rollout replica; 0 = 2 whenever at least 2 GPUs run (the layout the benchmark config names), 1 on a single GPU. "
                         "--rollout-tp 1 (one replica per GPU) is about 5 %% faster for this 7B model")
    ap.add_argument("--time-limit", type=float, default=790.0,
                    help="seconds of process wall clock the whole run may take: warm-up beyond three steps and timed steps that "
                         "would not fit are dropped and the JSON line reports the counts that ran; 0 = run exactly what was asked")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    single = int(os.environ.get("WORLD_SIZE", "1")) == 1
    if args.grad_ckpt < 0:
        args.grad_ckpt = 0
    if args.ref_offload < 0:
        # on one GPU the unsharded fp32 optimizer state (91 GB) leaves room for stored activations only if the frozen
        # reference weights wait in pinned host memory between their passes
        args.ref_offload = 1 if single and not args.grad_ckpt else 0
    if args.rollout_tp <= 0:
        args.rollout_tp = 1 if single else 2
    if args.token_budget <= 0:
        args.token_budget = 16384 if args.grad_ckpt else 8192
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "stocklibs":
        if not single:
            raise SystemExit("--impl stocklibs runs on one GPU")
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks"))
        import stocklibs_grpo

        stocklibs_grpo.run(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
