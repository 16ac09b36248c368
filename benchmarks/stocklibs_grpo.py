"""GRPO step built ONLY from the stock libraries the reference framework calls, on the same synthetic workload as
``bench.py``: vLLM for the rollout, Hugging Face ``transformers`` Qwen2 with FlashAttention-2 varlen for the two
log-prob passes and the update, ``torch.optim.AdamW`` for the optimizer. Nothing of ``verl_b200`` runs here (no model, no
kernel, no engine); it is the anchor the native number is compared with when the reference package itself cannot be
installed (it needs ray / tensordict / hydra, for which no offline wheels exist).

What it mirrors in the reference (paths inside the reference repository):

* rollout: ``verl/workers/rollout/vllm_rollout/vllm_async_server.py:484-536`` engine settings (``max_num_seqs``,
  ``gpu_memory_utilization``, prefix caching, CUDA graphs, sleep mode between rollouts), ``n`` samples per prompt;
* log-probs / update: ``verl/workers/engine/fsdp/transformer_impl.py:728-838`` — fp32 parameters with bf16 autocast
  (FSDP mixed precision param bf16 / reduce fp32), remove-padding packed micro-batches under a token budget,
  gradient checkpointing on (the reference default), grad-norm clip 1.0, AdamW;
* loss: ``verl/trainer/ppo/core_algos.py`` vanilla clip 0.2 + ``low_var_kl`` 1e-3, token-mean; GRPO advantages.

One process, one GPU. Per step: wake vLLM, push the actor's weights into it, generate, put it to sleep, old log-probs
(+ entropy), reference log-probs, advantages, 4 mini-batches of updates. Usage: ``python bench.py --impl stocklibs``.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import time


def _qwen2_config(args):
    from transformers import Qwen2Config

    presets = {"qwen2.5-7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
                                  num_key_value_heads=4, max_position_embeddings=32768, rope_theta=1000000.0, rms_norm_eps=1e-6,
                                  tie_word_embeddings=False),
               "tiny-qwen2": dict(vocab_size=2048, hidden_size=128, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                  num_key_value_heads=2, max_position_embeddings=2048, rope_theta=10000.0, rms_norm_eps=1e-6,
                                  tie_word_embeddings=True)}
    cfg = Qwen2Config(**presets[args.model], torch_dtype="bfloat16", architectures=["Qwen2ForCausalLM"], bos_token_id=None, eos_token_id=None,
                      pad_token_id=0, use_cache=False)
    return cfg


def _prompts(args, step: int, vocab_hi: int):
    import torch

    g = torch.Generator().manual_seed(1000 + step)
    lens = torch.randint(args.min_prompt, args.max_prompt + 1, (args.prompts_per_gpu,), generator=g)
    return [torch.randint(100, vocab_hi, (int(l),), generator=g).tolist() for l in lens]


def _micro_batches(lengths, budget):
    """Greedy first-fit over sequences sorted by length: lists of indices whose token counts stay under ``budget``."""
    order = sorted(range(len(lengths)), key=lambda i: lengths[i])
    out, cur, tok = [], [], 0
    for i in order:
        if cur and tok + lengths[i] > budget:
            out.append(cur)
            cur, tok = [], 0
        cur.append(i)
        tok += lengths[i]
    if cur:
        out.append(cur)
    return out


class _Timer:
    """CUDA events on a GPU, wall clock elsewhere (the CPU path only exists so that the training half can be tested)."""

    def __init__(self, cuda):
        import torch

        self.cuda = cuda
        self.t0 = time.perf_counter()
        if cuda:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.e0.record()

    def stop(self) -> float:
        import torch

        if self.cuda:
            self.e1.record()
            torch.cuda.synchronize()
            return self.e0.elapsed_time(self.e1) / 1000.0
        return time.perf_counter() - self.t0


def run(args, llm=None, sampling=None):
    """``llm`` / ``sampling``: a stand-in rollout engine for tests (same ``wake_up / sleep / generate / collective_rpc`` surface)."""
    import torch

    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")      # engine core in this process: weights can be pushed without IPC
    os.environ.setdefault("VLLM_ALLOW_INSECURE_SERIALIZATION", "1")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    t_start = time.time()
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(0)
    dev = torch.device("cuda" if cuda else "cpu")
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    attn_impl = "flash_attention_2" if cuda else "sdpa"
    cfg = _qwen2_config(args)
    model_dir = tempfile.mkdtemp(prefix="stocklibs_qwen2_")
    cfg.save_pretrained(model_dir)
    notes = {}
    n, R = args.n, args.response_length
    vocab_hi = min(150000, cfg.vocab_size)

    # ---------------------------------------------------------------- rollout engine (first, while the GPU is empty)
    if llm is None:
        from vllm import LLM, SamplingParams

        llm = LLM(model=model_dir, skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16", seed=0, gpu_memory_utilization=args.vllm_util,
                  max_num_seqs=args.prompts_per_gpu * n, max_model_len=args.max_prompt + R, enable_prefix_caching=True, enable_sleep_mode=True,
                  enforce_eager=False, generation_config="vllm", disable_log_stats=True)
        sp = SamplingParams(n=n, temperature=1.0, top_p=1.0, top_k=-1, max_tokens=R, detokenize=False, logprobs=0, seed=None)
    else:
        sp = sampling
    llm.sleep(level=1)
    if cuda:
        torch.cuda.empty_cache()         # what the engine's profiling run left in torch's caching allocator

    # ---------------------------------------------------------------- actor (fp32 + autocast), reference (bf16, frozen)
    from transformers import AutoModelForCausalLM

    torch.manual_seed(0)
    with torch.device(dev):
        actor = AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32, attn_implementation=attn_impl)
    actor.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
    actor.train()
    with torch.device(dev):
        ref = AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.bfloat16, attn_implementation=attn_impl)
    ref.load_state_dict({k: v.to(torch.bfloat16) for k, v in actor.state_dict().items()})
    ref.eval().requires_grad_(False)
    opt = torch.optim.AdamW(actor.parameters(), lr=1e-6, betas=(0.9, 0.999), weight_decay=0.01, fused=cuda)

    def push_weights():
        """Actor -> vLLM, every step (reference: per-tensor stream into ``load_weights``)."""
        def load(worker):
            worker.model_runner.model.load_weights((k, v.detach().to(torch.bfloat16)) for k, v in actor.state_dict().items())
            return True
        try:
            llm.collective_rpc(load)
            notes.setdefault("weight_sync", "actor state_dict -> vLLM load_weights each step")
        except Exception as e:  # noqa: BLE001
            notes["weight_sync"] = f"skipped ({type(e).__name__}: {str(e)[:120]}); the rollout keeps its initial weights, which only lowers this arm's step time"

    def forward_logprobs(model, ids_list, resp_lens, need_entropy, grad):
        """Packed forward of whole sequences; returns per-sequence log-probs (and entropies) of the response tokens."""
        lens = [len(x) for x in ids_list]
        flat = torch.tensor([t for x in ids_list for t in x], device=dev, dtype=torch.long)[None]
        pos = torch.cat([torch.arange(l, device=dev) for l in lens])[None]
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=dev, dtype=torch.int32)
        kw = dict(cu_seq_lens_q=cu, cu_seq_lens_k=cu, max_length_q=max(lens), max_length_k=max(lens))
        with torch.autocast(dev.type, dtype=torch.bfloat16), torch.set_grad_enabled(grad):
            logits = model(input_ids=flat, position_ids=pos, use_cache=False, **kw).logits[0]
        logits = logits.float() / 1.0                      # temperature 1.0
        lse = torch.logsumexp(logits, -1)
        tgt = torch.roll(flat[0], -1)
        lp_all = logits.gather(1, tgt[:, None])[:, 0] - lse
        ent_all = None
        if need_entropy:
            p = torch.softmax(logits, -1)
            ent_all = lse - (p * logits).sum(-1)
        outs, ents, off = [], [], 0
        for l, r in zip(lens, resp_lens):
            outs.append(lp_all[off + l - r - 1: off + l - 1])
            if ent_all is not None:
                ents.append(ent_all[off + l - r - 1: off + l - 1])
            off += l
        return outs, ents

    def step(s: int):
        t = {}
        t0 = time.perf_counter()
        prompts = _prompts(args, s, vocab_hi)
        opt.zero_grad(set_to_none=True)
        if cuda:
            torch.cuda.empty_cache()     # gradients and activations of the last update: the KV cache needs the room back
        llm.wake_up()
        push_weights()
        outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, use_tqdm=False)
        seqs, resp_lens = [], []
        for p, o in zip(prompts, outs):
            for c in o.outputs:
                seqs.append(p + list(c.token_ids))
                resp_lens.append(len(c.token_ids))
        llm.sleep(level=1)
        if cuda:
            torch.cuda.empty_cache()
        sync()
        t["gen"] = time.perf_counter() - t0
        lens = [len(x) for x in seqs]
        # rule reward: 1 if last response token id mod 7 == (sum of prompt ids) mod 7
        rewards = torch.tensor([1.0 if (seqs[i][-1] % 7) == (sum(prompts[i // n]) % 7) else 0.0 for i in range(len(seqs))])
        grp = rewards.view(-1, n)
        adv = ((grp - grp.mean(1, keepdim=True)) / (grp.std(1, keepdim=True) + 1e-6)).view(-1).to(dev)
        t1 = time.perf_counter()
        old, refs = [None] * len(seqs), [None] * len(seqs)
        for mb in _micro_batches(lens, 2 * args.token_budget):
            lp, _ = forward_logprobs(actor, [seqs[i] for i in mb], [resp_lens[i] for i in mb], True, False)
            for i, x in zip(mb, lp):
                old[i] = x
        sync()
        t["old_log_prob"] = time.perf_counter() - t1
        t1 = time.perf_counter()
        for mb in _micro_batches(lens, 2 * args.token_budget):
            lp, _ = forward_logprobs(ref, [seqs[i] for i in mb], [resp_lens[i] for i in mb], False, False)
            for i, x in zip(mb, lp):
                refs[i] = x
        sync()
        t["ref"] = time.perf_counter() - t1
        t1 = time.perf_counter()
        mini = args.mini_prompts_per_gpu * n
        loss_val = 0.0
        for m0 in range(0, len(seqs), mini):
            idx = list(range(m0, min(len(seqs), m0 + mini)))
            tok_total = float(sum(resp_lens[i] for i in idx))
            opt.zero_grad(set_to_none=True)
            for mb in _micro_batches([lens[i] for i in idx], args.token_budget):
                mb = [idx[j] for j in mb]
                lp, _ = forward_logprobs(actor, [seqs[i] for i in mb], [resp_lens[i] for i in mb], False, True)
                new = torch.cat(lp)
                o = torch.cat([old[i] for i in mb])
                rf = torch.cat([refs[i] for i in mb])
                a = torch.cat([adv[i].expand(resp_lens[i]) for i in mb])
                ratio = torch.exp(new - o)
                pg = torch.maximum(-a * ratio, -a * ratio.clamp(0.8, 1.2))
                d = rf - new
                kl = (torch.exp(d) - d - 1).clamp(-10, 10)
                loss = (pg + 1e-3 * kl).sum() / tok_total
                loss.backward()
                loss_val += float(loss.detach())
            torch.nn.utils.clip_grad_norm_(actor.parameters(), 1.0)
            opt.step()
        sync()
        t["update_actor"] = time.perf_counter() - t1
        t["step"] = time.perf_counter() - t0
        return sum(lens), t, loss_val

    warm = []
    for w in range(args.warmup):
        _, t, _ = step(w)
        warm.append(round(t["step"], 3))
        if args.verbose:
            print(f"[stocklibs warmup {w}] {t}", file=sys.stderr, flush=True)
        if args.time_limit > 0 and w + 1 >= 3 and time.time() - t_start + t["step"] * (args.warmup - w - 1 + args.steps) > args.time_limit:
            break
    steps = args.steps
    if args.time_limit > 0 and warm:
        steps = max(1, min(args.steps, int((args.time_limit - (time.time() - t_start)) // (max(warm[1:] or warm) * 1.03))))
    sync()
    timer = _Timer(cuda)
    tw0 = time.perf_counter()
    tokens, per = 0, []
    for s in range(steps):
        nt, t, _ = step(len(warm) + s)
        tokens += nt
        per.append({k: round(v, 3) for k, v in t.items()})
        if args.verbose:
            print(f"[stocklibs step {s}] {t}", file=sys.stderr, flush=True)
    dev_s = timer.stop()
    wall = time.perf_counter() - tw0
    import transformers

    try:
        import vllm

        vllm_version = vllm.__version__
    except Exception:  # noqa: BLE001
        vllm_version = None

    out = {"metric": "GRPO step tokens/s (rollout+train), Qwen2.5-7B arch", "value": tokens / dev_s, "unit": "tokens/s", "n_gpus": 1, "steps": steps,
           "warmup": len(warm), "steps_requested": args.steps, "warmup_requested": args.warmup, "ms_per_step": dev_s * 1000.0 / steps,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic prompts, random-init weights",
           "impl": "stocklibs",
           "config": {"model": args.model, "global_batch": f"{args.prompts_per_gpu} prompts x n={n}",
                      "seq_len": f"prompt U[{args.min_prompt},{args.max_prompt}] + response <= {R}",
                      "parallelism": "1 GPU: vLLM engine (sleep mode) + transformers fp32 params with bf16 autocast, FlashAttention-2 varlen, torch AdamW",
                      "libraries": {"vllm": vllm_version, "transformers": transformers.__version__, "torch": torch.__version__},
                      "gradient_checkpointing": True, "token_budget_per_micro_batch": args.token_budget, "notes": notes},
           "e2e": {"value": tokens / wall, "unit": "tokens/s"},
           "step_breakdown_s": {k: [d.get(k) for d in per] for k in per[0]} if per else {},
           "warmup_step_s": warm, "tokens_per_step": tokens / max(1, steps), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 1) if cuda else None}
    print(json.dumps(out), flush=True)
    return out
