"""In-house rollout engine: paged-KV continuous-batching generation on the training process's own weights.

It replaces the vLLM / SGLang servers of the reference (``verl/workers/rollout/vllm_rollout/vllm_async_server.py``,
``verl/workers/rollout/replica.py``). Design points for a B200:

* **Zero-copy weights.** The engine reads the trainer's resident bf16 parameters; "weight sync" for a colocated
  TP=1 replica is a no-op (the reference all-gathers every tensor and ships it through CUDA IPC,
  ``verl/workers/engine_workers.py:734-836``).
* **Static decode batch + CUDA graph.** A decode step always runs over all ``max_num_seqs`` slots with device-side
  position / slot bookkeeping, so one captured graph serves every step; idle slots have kv_len 0.
* **Prompt sharing.** The n samples of a GRPO prompt prefill once; siblings fork the prompt's KV blocks by reference.
* **Lazy EOS detection.** Sampled tokens are kept on the device and read back every ``sync_interval`` steps, so the
  host never blocks on a decode step.
"""

from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from verl_b200 import ops
from verl_b200.models.transformer import DecoderLM
from verl_b200.ops import _ext
from verl_b200.ops.attention import build_tile_tables, paged_decode_attention
from verl_b200.workers.rollout.scheduler import STEP_DECODE, STEP_IDLE, STEP_PREFILL, Scheduler

__all__ = ["SamplingParams", "TokenOutput", "InferenceEngine", "BLOCK_SIZE"]

BLOCK_SIZE = 64


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    max_tokens: int = 1024
    ignore_eos: bool = False
    logprobs: bool = True
    top_logprobs: int = 0      # also return the k most likely tokens (ids + log-probs) at every step (score centering)
    # >= 0: score the prompt instead of generating — per position the log-prob of the k most likely tokens under the context before it
    # (0: only the log-prob of the token that is there). What a distillation teacher is asked for.
    prompt_logprobs: int = -1
    seed: int = 0
    stop_token_ids: Sequence[int] = ()


@dataclass
class TokenOutput:
    """Result of one generation request (same fields as the reference's ``TokenOutput``, rollout/replica.py:34-46)."""

    token_ids: list
    log_probs: Optional[list] = None
    top_ids: Optional[list] = None           # [steps][k] with SamplingParams.top_logprobs = k
    top_log_probs: Optional[list] = None
    routed_experts: Optional[np.ndarray] = None
    stop_reason: Optional[str] = None
    num_preempted: int = 0
    extra_fields: dict = field(default_factory=dict)


def _sample_reference(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, gen: torch.Generator):
    """PyTorch oracle of the sampling kernel (exact sort-based top-k / top-p)."""
    x = logits.float()
    if temperature <= 0:
        tok = x.argmax(-1)
        lp = torch.log_softmax(x, -1).gather(-1, tok[:, None]).squeeze(-1)
        return tok, lp
    x = x / temperature
    if top_k and 0 < top_k < x.shape[-1]:
        kth = torch.topk(x, top_k, dim=-1).values[:, -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p < 1.0:
        sx, si = torch.sort(x, dim=-1, descending=True)
        cp = torch.softmax(sx, -1).cumsum(-1)
        drop = cp - torch.softmax(sx, -1) >= top_p
        sx = sx.masked_fill(drop, float("-inf"))
        x = torch.full_like(x, float("-inf")).scatter(-1, si, sx)
    logp = torch.log_softmax(x, -1)
    tok = torch.multinomial(logp.exp(), 1, generator=gen).squeeze(-1)
    return tok, logp.gather(-1, tok[:, None]).squeeze(-1)


class InferenceEngine:
    def __init__(self, model: DecoderLM, max_num_seqs: int = 256, max_model_len: int = 2048, num_blocks: Optional[int] = None,
                 max_num_batched_tokens: int = 8192, gpu_memory_utilization: float = 0.5, enforce_eager: bool = False,
                 sync_interval: int = 16, enable_prefix_sharing: bool = True, decode_splits: int = 0, tp_group=None, tp_ctx=None,
                 quantization: Optional[str] = None, enable_chunked_prefill: bool = True, enable_prefix_caching: bool = True):
        """``model`` may be a vision-language model (``verl_b200.models.vision.VisionLanguageModel``): its decoder serves the
        tokens, its tower embeds the images of multimodal requests at prefill.
        ``tp_group`` / ``tp_ctx``: tensor-parallel replica. ``model`` is then this rank's slice (``build_rollout_shard``); every
        rank of the group runs the same requests in lockstep (same scheduler decisions, same sampled tokens) and the
        row-parallel projections end in an all-reduce — fused into the GEMM epilogue over NVLink peer memory when
        ``tp_ctx`` (a ``TPContext``) is given, NCCL otherwise.
        ``enable_chunked_prefill``: prompts longer than ``max_num_batched_tokens`` are computed in chunks of that size, each
        attending to the chunks already in the paged cache, so no step exceeds the token budget. ``enable_prefix_caching``:
        full KV blocks stay findable by a hash of their tokens and later requests that begin with the same tokens (the next
        turn of a conversation, a shared system prompt) compute only the rest. ``enable_prefix_sharing`` is the cheaper
        special case for the n samples of one prompt submitted together (reference knobs: ``enable_chunked_prefill`` /
        ``enable_prefix_caching`` / ``max_num_batched_tokens`` of verl/trainer/config/rollout/rollout.yaml)."""
        self.visual = self.vision_config = None
        if hasattr(model, "visual") and hasattr(model, "language_model"):
            self.visual, self.vision_config, model = model.visual, model.vcfg, model.language_model
        self.model = model
        sw = int(getattr(getattr(model, "cfg", None), "sliding_window", 0) or 0)
        if sw and max_model_len > sw:
            raise NotImplementedError(f"this checkpoint uses sliding-window attention over {sw} tokens; max_model_len={max_model_len} would need "
                                      "windowed decode attention, which is not built")
        if getattr(model, "lora_config", None) and (quantization or tp_group is not None):
            raise NotImplementedError("adapters are served unmerged only by bf16 replicas without tensor parallelism; give the engine a merged copy instead")
        if getattr(getattr(model, "cfg", None), "mlp_act", "swiglu") != "swiglu" and (quantization or tp_group is not None):
            raise NotImplementedError("models with an un-gated MLP (Apertus) run in the rollout engine without tensor parallelism or fp8 weights")
        self.tp_group, self.tp = tp_group, tp_ctx
        # "fp8": W8A8 projections (per-output-channel e4m3 weights re-quantised from the live bf16 weights at every wake_up,
        # per-token e4m3 activations, tcgen05 f8f6f4 GEMM); embeddings, norms, lm_head and the KV cache stay bf16.
        # Reference: FP8 rollout, verl/utils/fp8_utils.py + verl/utils/kernel/fp8_kernel.py (weights quantised during sync).
        # "fp8_block": the same with 128x128 weight blocks and 1x128 activation groups (the block-scaled GEMM)
        assert quantization in (None, "", "fp8", "fp8_block"), f"unsupported rollout quantization {quantization!r}"
        self.quantization = quantization or None
        self._w8: dict = {}
        self.cfg = model.cfg
        self.device = model.embed_tokens.device
        self.dtype = model.embed_tokens.dtype
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.max_blocks_per_seq = (max_model_len + BLOCK_SIZE - 1) // BLOCK_SIZE + 1
        self.max_num_batched_tokens = max_num_batched_tokens
        self.gpu_memory_utilization = gpu_memory_utilization
        self.enforce_eager = enforce_eager or self.device.type != "cuda"
        self.sync_interval = max(1, sync_interval)
        self.enable_prefix_sharing = enable_prefix_sharing
        self.enable_chunked_prefill, self.enable_prefix_caching = bool(enable_chunked_prefill), bool(enable_prefix_caching)
        self.native = self.device.type == "cuda" and self.dtype == torch.bfloat16 and _ext.available()
        self._num_blocks_cfg = num_blocks
        self.cache: Optional[torch.Tensor] = None
        self.sched: Optional[Scheduler] = None
        self._graph = None
        self.decode_splits = decode_splits
        self._cpu_gen = torch.Generator(device="cpu")
        self.stats = {"prefill_tokens": 0, "decode_steps": 0, "preemptions": 0, "forked": 0, "t_prefill": 0.0, "t_capture": 0.0,
                      "t_decode": 0.0, "t_flush": 0.0, "t_wake": 0.0, "prefix_cache_hit_tokens": 0, "prefill_chunks": 0}
        self.profile = False   # when set, phases are bracketed by device synchronisations and timed
        # router replay (R3): record the experts every fed token was routed to, per layer, and return them with the tokens
        # (reference: vLLM ``enable_return_routed_experts``, verl/workers/rollout/vllm_rollout/vllm_async_server.py:440-454,745-747)
        self.record_routing = False
        self._last_routed: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ memory lifecycle (sleep / wake_up)
    def _decide_num_blocks(self) -> int:
        if self._num_blocks_cfg:
            return int(self._num_blocks_cfg)
        c = self.cfg
        per_block = c.num_hidden_layers * 2 * c.num_key_value_heads * BLOCK_SIZE * c.head_dim * self.model.embed_tokens.element_size()
        want = self.max_num_seqs * self.max_blocks_per_seq + 1
        if self.device.type == "cuda":
            torch.cuda.empty_cache()          # memory cached by the training phase must count as free
            free, total = torch.cuda.mem_get_info(self.device)
            budget = min(free * 0.9, total * self.gpu_memory_utilization)
            got = min(want, max(int(budget // per_block), self.max_blocks_per_seq + 2))
            if got < want:
                print(f"[rollout] KV cache limited to {got} blocks ({got * per_block / 2**30:.1f} GiB) of the {want} needed to hold "
                      f"{self.max_num_seqs} sequences of {self.max_model_len} tokens; expect preemptions", flush=True)
            want = got
        if self.tp_group is not None:
            # every rank of a tensor-parallel replica must run the same schedule: agree on the smallest cache
            import torch.distributed as dist

            t = torch.tensor([want], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.tp_group)
            want = int(t.item())
        return want

    def _tick(self):
        import time

        if self.profile and self.device.type == "cuda":
            torch.cuda.synchronize()
        return time.perf_counter()

    def wake_up(self):
        """Allocate the KV cache and the static decode buffers."""
        if self.cache is not None:
            return
        t0 = self._tick()
        try:
            self._wake_up_impl()
        finally:
            self.stats["t_wake"] += self._tick() - t0

    def _quantise_weights(self):
        """(Re)build the e4m3 copies of the dense projection weights from the current bf16 weights."""
        self._w8 = {}
        if self.quantization not in ("fp8", "fp8_block") or not self.native or self.tp_group is not None:
            return
        from verl_b200.ops.quant import blockwise_cast_to_fp8, rowwise_cast_to_fp8

        cast = rowwise_cast_to_fp8 if self.quantization == "fp8" else blockwise_cast_to_fp8

        for layer in self.model.layers:
            ws = [layer.self_attn.qkv_proj, layer.self_attn.o_proj]
            if not self.cfg.is_moe:
                ws += [layer.mlp.gate_up_proj, layer.mlp.down_proj]
            for w in ws:
                self._w8[id(w)] = cast(w.detach())

    def _linear(self, x: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
        q = self._w8.get(id(w))
        if q is None:
            return ops.linear(x, w, bias)
        from verl_b200.ops.quant import fp8_block_linear, fp8_linear

        return (fp8_linear if self.quantization == "fp8" else fp8_block_linear)(x, q[0], q[1], bias)

    def _lora_delta(self, mod, name: str, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """Low-rank adapters are served as they are trained: ``y + scale * (x A^T) B^T`` from the trainer's live adapter tensors, so
        a LoRA policy needs no merged copy of the weights and no weight hand-off (reference: LoRA adapters loaded into the serving
        engine instead of merged weights, verl/workers/rollout/vllm_rollout ``load_format`` / ``lora`` paths)."""
        ad = getattr(mod, "_lora", None)
        if not ad or name not in ad:
            return y
        a_name, b_name, scale = ad[name]
        return y + scale * ops.linear(ops.linear(x, getattr(mod, a_name)), getattr(mod, b_name))

    def _wake_up_impl(self):
        c = self.cfg
        self._quantise_weights()
        nb = self._decide_num_blocks()
        self.num_blocks = nb
        # zero-filled: masked (probability 0) positions still enter the P·V product, so they must hold finite values
        self.cache = torch.zeros(c.num_hidden_layers, nb, 2, c.num_key_value_heads, BLOCK_SIZE, c.head_dim, dtype=self.dtype,
                                 device=self.device)
        S, dev = self.max_num_seqs, self.device
        self.cur_tokens = torch.zeros(S, dtype=torch.int64, device=dev)
        self.positions = torch.zeros(S, dtype=torch.int32, device=dev)
        self.rope_delta = torch.zeros(S, dtype=torch.int32, device=dev)      # multimodal prompts: rotary position − cache position
        self.active = torch.zeros(S, dtype=torch.int32, device=dev)
        self.block_table = torch.zeros(S, self.max_blocks_per_seq, dtype=torch.int32, device=dev)
        self.kv_lens = torch.zeros(S, dtype=torch.int32, device=dev)
        self.rng = torch.zeros(2, dtype=torch.int64, device=dev)
        self.row_ids = torch.arange(S, dtype=torch.int32, device=dev)
        self.out_tok = torch.zeros(S, dtype=torch.int64, device=dev)
        self.out_lp = torch.zeros(S, dtype=torch.float32, device=dev)
        K = self.sync_interval
        self.hist_tok = torch.zeros(K, S, dtype=torch.int64, device=dev)
        self.hist_lp = torch.zeros(K, S, dtype=torch.float32, device=dev)
        self.hist_idx = torch.zeros(1, dtype=torch.int64, device=dev)
        self.block_table_host = np.zeros((S, self.max_blocks_per_seq), dtype=np.int32)
        pin = self.device.type == "cuda"
        self._bt_pinned = [torch.zeros(S, self.max_blocks_per_seq, dtype=torch.int32, pin_memory=pin) for _ in range(4)]
        self._bt_events = [None] * 4
        self._bt_ring = 0
        if self.decode_splits <= 0:
            # enough CTAs to fill the machine: B * Hkv * splits >= ~2 waves of 148 SMs
            self.decode_splits = max(1, min(8, (296 + S * c.num_key_value_heads - 1) // (S * c.num_key_value_heads)))
        self.workspace = torch.empty(S * c.num_attention_heads * self.decode_splits * 130, dtype=torch.float32, device=dev) \
            if self.decode_splits > 1 else None
        self.sched = Scheduler(nb, BLOCK_SIZE, S, self.max_num_batched_tokens, chunked_prefill=self.enable_chunked_prefill,
                               prefix_caching=self.enable_prefix_caching)
        self._sched_counted = [0, 0]
        self._graph = None

    def sleep(self):
        """Release the KV cache and graphs so training can use the memory (reference: rollout ``sleep``/``release``)."""
        self._graph = None
        self.cache = None
        self.sched = None
        self.workspace = None
        self._w8 = {}
        for n in ("hist_tok", "hist_lp", "hist_routed", "block_table", "cur_tokens", "positions", "kv_lens", "active"):
            if hasattr(self, n):
                delattr(self, n)
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    # ------------------------------------------------------------------ model forward (shared by prefill and decode)
    def _layer_stack(self, tokens, positions, slots, attn_fn, rope=None, visual=None):
        """Runs embedding → layers → final norm; ``attn_fn(layer_idx, qkv)`` returns the attention output. ``rope``: per-token
        (cos, sin) tables replacing the position-indexed ones (multimodal rotary embedding, ``positions`` = row numbers);
        ``visual``: (row indices, embeddings) that replace the image placeholder tokens' embeddings."""
        m, c = self.model, self.cfg
        cos, sin = rope if rope is not None else m.rope(self.device)
        h = m.embed_tokens.index_select(0, tokens)
        if visual is not None:
            h = h.index_copy(0, visual[0], visual[1].to(h.dtype))
        res = None
        n_rot = c.num_attention_heads + c.num_key_value_heads
        record = self.record_routing and c.is_moe
        routed = []
        for li, layer in enumerate(m.layers):
            if res is None:
                res = h
                x = ops.rmsnorm(h, layer.input_layernorm, c.rms_norm_eps)
            else:
                x, res = ops.add_rmsnorm(h, res, layer.input_layernorm, c.rms_norm_eps)
            at = layer.self_attn
            qkv = self._lora_delta(at, "qkv_proj", x, self._linear(x, at.qkv_proj, at.qkv_bias))
            if c.qk_norm:
                T = qkv.shape[0]
                q, k, v = qkv.split([c.q_size, c.kv_size, c.kv_size], dim=-1)
                q = ops.rmsnorm(q.reshape(-1, c.head_dim), at.q_norm, c.rms_norm_eps).reshape(T, c.q_size)
                k = ops.rmsnorm(k.reshape(-1, c.head_dim), at.k_norm, c.rms_norm_eps).reshape(T, c.kv_size)
                qkv = torch.cat([q, k, v], dim=-1)
            qkv = ops.apply_rope_(qkv, positions, cos, sin, n_rot, c.head_dim)
            self._cache_write(li, qkv, slots)
            o = attn_fn(li, qkv)
            a = self._lora_delta(at, "o_proj", o, self._row_parallel(o, at.o_proj))
            x, res = ops.add_rmsnorm(a, res, layer.post_attention_layernorm, c.rms_norm_eps)
            if self.tp_group is not None and not c.is_moe:
                h = self._row_parallel(ops.swiglu(ops.linear(x, layer.mlp.gate_up_proj)), layer.mlp.down_proj)
            elif self._w8 and not c.is_moe:
                h = self._linear(ops.swiglu(self._linear(x, layer.mlp.gate_up_proj)), layer.mlp.down_proj)
            else:
                if record:
                    layer.mlp.record_routing = True
                h = layer.mlp(x)
                if record:
                    routed.append(layer.mlp.last_topk)
            if visual is not None and len(visual) > 2 and visual[2] is not None and li < len(visual[2]):
                h = h.index_add(0, visual[0], visual[2][li].to(h.dtype))       # deep-stack vision features join the stream (h + res)
        self._last_routed = torch.stack(routed, 1).to(torch.int16) if record else None      # [T, layers, topk]
        return ops.add_rmsnorm(h, res, m.norm, c.rms_norm_eps)[0]

    def _tp_sync_samples(self, tok: torch.Tensor, lp: torch.Tensor) -> None:
        """The ranks of a tensor-parallel replica compute identical logits and draw with identical random streams, but the
        schedule (who finished, who is admitted) must never depend on that staying bit-exact: the first rank's tokens are
        the replica's tokens."""
        if self.tp_group is None:
            return
        import torch.distributed as dist

        src = dist.get_global_rank(self.tp_group, 0)
        dist.broadcast(tok, src=src, group=self.tp_group)
        dist.broadcast(lp, src=src, group=self.tp_group)

    def _row_parallel(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``x @ wᵀ`` summed over the tensor-parallel ranks (plain GEMM when the replica is a single GPU)."""
        if self.tp_group is None:
            return self._linear(x, w)
        if self.tp is not None:
            return self.tp.gemm_allreduce(x.contiguous(), w)
        import torch.distributed as dist

        y = ops.linear(x, w).contiguous()
        dist.all_reduce(y, group=self.tp_group)
        return y

    def _cache_write(self, li: int, qkv: torch.Tensor, slots: torch.Tensor):
        c = self.cfg
        if self.native and c.head_dim == 128:
            _ext.ops().kv_cache_write(qkv, slots, self.cache[li], c.num_attention_heads, c.num_key_value_heads)
            return
        T = qkv.shape[0]
        k = qkv[:, c.q_size : c.q_size + c.kv_size].reshape(T, c.num_key_value_heads, c.head_dim)
        v = qkv[:, c.q_size + c.kv_size :].reshape(T, c.num_key_value_heads, c.head_dim)
        ok = slots >= 0
        blk, off = (slots[ok] // BLOCK_SIZE), (slots[ok] % BLOCK_SIZE)
        self.cache[li, blk, 0, :, off] = k[ok]
        self.cache[li, blk, 1, :, off] = v[ok]

    def _sample(self, logits, temperature, top_k, top_p, row_ids=None, out_tok=None, out_lp=None):
        B = logits.shape[0]
        if out_tok is None:
            out_tok = torch.empty(B, dtype=torch.int64, device=logits.device)
            out_lp = torch.empty(B, dtype=torch.float32, device=logits.device)
        if self.native:
            _ext.ops().sample(logits, float(temperature), int(top_k if top_k else -1), float(top_p), self.rng, row_ids, out_tok, out_lp)
        else:
            t, lp = _sample_reference(logits.cpu(), temperature, top_k, top_p, self._cpu_gen)
            out_tok.copy_(t)
            out_lp.copy_(lp)
        return out_tok, out_lp

    # ------------------------------------------------------------------ prefill
    def _push_block_table(self):
        i = self._bt_ring
        self._bt_ring = (i + 1) % len(self._bt_pinned)
        if self._bt_events[i] is not None:
            self._bt_events[i].synchronize()
        self._bt_pinned[i].copy_(torch.from_numpy(self.block_table_host))
        self.block_table.copy_(self._bt_pinned[i], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._bt_events[i] = ev

    def _prefill(self, seqs: list, sp: SamplingParams):
        """``seqs``: list of (request, slot, start, n): compute tokens ``[start, start + n)`` of prompt + anything generated
        before a preemption; the tokens before ``start`` are in the paged cache already (prefix-cache hits or earlier chunks of
        a long prompt). Returns (logits of the sequences whose prompt is complete after this step, their indices in ``seqs``)."""
        c = self.cfg
        toks, pos, slots, lens, starts, pre_blk, pre_off, final = [], [], [], [], [], [], [], []
        for i, (req, slot, start, n) in enumerate(seqs):
            ids = req["prompt"] + req["out"]
            blocks = self.sched.blocks(req["id"])
            self.block_table_host[slot, : len(blocks)] = blocks
            self.block_table_host[slot, len(blocks):] = 0
            p = np.arange(start, start + n)
            toks.append(np.asarray(ids[start:start + n], dtype=np.int64))
            pos.append(p.astype(np.int32))
            slots.append(blocks[p // BLOCK_SIZE].astype(np.int64) * BLOCK_SIZE + p % BLOCK_SIZE)
            lens.append(n)
            starts.append(start)
            if start:
                pp = np.arange(start)
                pre_blk.append(blocks[pp // BLOCK_SIZE].astype(np.int64))
                pre_off.append((pp % BLOCK_SIZE).astype(np.int64))
            if start + n == len(ids):
                final.append(i)
        dev = self.device
        tokens = torch.from_numpy(np.concatenate(toks)).to(dev)
        positions = torch.from_numpy(np.concatenate(pos)).to(dev)
        slot_map = torch.from_numpy(np.concatenate(slots)).to(dev)
        cu_cpu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu_cpu[1:] = torch.cumsum(torch.tensor(lens), 0)
        cu = cu_cpu.to(dev)
        max_len = max(lens)

        if not any(starts):
            def attn(li, qkv):
                return ops.attention_varlen(qkv, cu, c.num_attention_heads, c.num_key_value_heads, c.head_dim, max_len, cu_cpu)
        else:
            # some sequences continue from cached tokens: attention runs on an expanded layout in which every such sequence is
            # preceded by its cached K/V rows (gathered from the paged cache, queries left at zero); the kernels skip the query
            # tiles that lie entirely inside those rows
            exp_lens = [st + n for st, n in zip(starts, lens)]
            cu_exp_cpu = torch.zeros(len(lens) + 1, dtype=torch.int32)
            cu_exp_cpu[1:] = torch.cumsum(torch.tensor(exp_lens), 0)
            base = cu_exp_cpu[:-1].tolist()
            q_pos = torch.from_numpy(np.concatenate([np.arange(b + st, b + st + n) for b, st, n in zip(base, starts, lens)])).to(dev)
            pre_pos = torch.from_numpy(np.concatenate([np.arange(b, b + st) for b, st in zip(base, starts) if st])).to(dev)
            blk_i, off_i = torch.from_numpy(np.concatenate(pre_blk)).to(dev), torch.from_numpy(np.concatenate(pre_off)).to(dev)
            cu_exp, E, max_exp, q_starts = cu_exp_cpu.to(dev), int(cu_exp_cpu[-1]), max(exp_lens), tuple(starts)

            def attn(li, qkv):
                kv = self.cache[li][blk_i, :, :, off_i]                          # [rows, 2, Hkv, D]: K heads then V heads of each row
                qkv_exp = qkv.new_zeros(E, qkv.shape[1])
                qkv_exp.index_copy_(0, q_pos, qkv)
                qkv_exp[pre_pos, c.q_size:] = kv.reshape(kv.shape[0], -1)
                o = ops.attention_varlen(qkv_exp, cu_exp, c.num_attention_heads, c.num_key_value_heads, c.head_dim, max_exp, cu_exp_cpu,
                                         q_starts=q_starts)
                return o.index_select(0, q_pos)

        rope = visual = None
        if self.visual is not None and any(req.get("mm") for req, *_ in seqs):
            rope, visual = self._multi_modal_prefill([req for req, *_ in seqs], tokens)
            positions = torch.arange(tokens.shape[0], dtype=torch.int32, device=dev)
        h = self._layer_stack(tokens, positions, slot_map, attn, rope, visual)
        self.stats["prefill_tokens"] += int(sum(lens))
        if self._last_routed is not None:
            # a (re)prefill from token 0 starts the request's routing record over; later chunks extend it
            rt = self._last_routed.cpu().numpy()
            off = 0
            for (req, _, start, _n), L in zip(seqs, lens):
                if start == 0:
                    req["routed"] = [rt[off:off + L]]
                else:
                    req.setdefault("routed", []).append(rt[off:off + L])
                off += L
        if not final:
            return None, final
        last = (cu[1:] - 1).long().index_select(0, torch.tensor(final, device=dev))
        logits = ops.linear(h.index_select(0, last), self.model.output_weight)
        return logits, final

    def _multi_modal_prefill(self, reqs: list, tokens: torch.Tensor):
        """Vision-language prompts: per-token rotary tables from the 3-stream positions of every sequence, and the vision
        tower's rows for the image placeholder tokens (reference: the multi_modal_data path of the serving engines,
        verl/workers/rollout/vllm_rollout/vllm_async_server.py:561-640)."""
        from verl_b200.models.vision import get_rope_index, mrope_tables

        v, c = self.vision_config, self.cfg
        pos3, pix, grids = [], [], []
        for req in reqs:
            mm = req.get("mm") or {}
            g = mm.get("image_grid_thw")
            p, _ = get_rope_index(torch.as_tensor(req["prompt"] + req["out"]), g, v, grid_t_scale=mm.get("grid_t_scale"))
            pos3.append(p)
            if g is not None and len(g):
                pix.append(torch.as_tensor(mm["pixel_values"]))
                grids.append(torch.as_tensor(g).reshape(-1, 3))
        rope = mrope_tables(torch.cat(pos3, 1).to(self.device), c.head_dim, c.rope_theta, v.mrope_section, getattr(v, "mrope_interleaved", False))
        visual = None
        if pix:
            rows = self.visual(torch.cat(pix, 0).to(self.device), torch.cat(grids, 0))
            idx = ((tokens == v.image_token_id) | (tokens == v.video_token_id)).nonzero(as_tuple=True)[0]
            assert idx.numel() == rows.shape[0], f"{idx.numel()} image placeholder tokens but {rows.shape[0]} merged patch embeddings"
            # Qwen3-VL: the tower also leaves one feature set per deep-stack block, added to the stream after the first decoder layers
            deep = list(self.visual.last_deepstack) if getattr(v, "variant", "") == "qwen3_vl" else None
            visual = (idx, rows, deep)
        return rope, visual

    def _start_sequences(self, reqs_slots: list, logits: torch.Tensor, sp: SamplingParams):
        """Sample the first new token of each sequence from its last-prompt-token logits and arm its decode slot."""
        slots = torch.tensor([s for _, s in reqs_slots], dtype=torch.int64, device=self.device)
        rid = slots.to(torch.int32)
        tok, lp = self._sample(logits, sp.temperature, sp.top_k, sp.top_p, row_ids=rid)
        self._tp_sync_samples(tok, lp)
        if self.native:
            self.rng[1] += 1
        plen = torch.tensor([len(r["prompt"]) + len(r["out"]) for r, _ in reqs_slots], dtype=torch.int32, device=self.device)
        self.cur_tokens.index_copy_(0, slots, tok)
        self.positions.index_copy_(0, slots, plen)
        if self.visual is not None:      # multimodal prompts: generated tokens continue after the image grid, not after its token count
            delta = torch.tensor([int(r.get("rope_delta", 0)) for r, _ in reqs_slots], dtype=torch.int32, device=self.device)
            self.rope_delta.index_copy_(0, slots, delta)
        self.kv_lens.index_copy_(0, slots, plen)
        self.active.index_fill_(0, slots, 1)
        tok_h, lp_h = tok.tolist(), lp.tolist()
        top = None
        if sp.top_logprobs > 0:
            tv, ti = self._top_head(logits, sp)
            top = (ti.tolist(), tv.tolist())
        for j, ((req, _), t, l) in enumerate(zip(reqs_slots, tok_h, lp_h)):
            req["out"].append(int(t))
            req["lp"].append(float(l))
            if top is not None:
                req.setdefault("topi", []).append(top[0][j])
                req.setdefault("topv", []).append(top[1][j])
            req["n_gen"] = len(req["out"])

    @staticmethod
    def _top_head(logits: torch.Tensor, sp: SamplingParams):
        """(log-probs [B, k], ids [B, k]) of the k most likely tokens under the sampling temperature."""
        lsm = torch.log_softmax(logits.float() / max(float(sp.temperature), 1e-6), dim=-1)
        return lsm.topk(int(sp.top_logprobs), dim=-1)

    def _ensure_top_hist(self, k: int):
        if getattr(self, "hist_topi", None) is None or self.hist_topi.shape[-1] != k:
            K, S = self.hist_tok.shape
            self.hist_topi = torch.zeros(K, S, k, dtype=torch.int64, device=self.device)
            self.hist_topv = torch.zeros(K, S, k, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ decode
    def _decode_body(self, sp: SamplingParams):
        """One token for every slot. All bookkeeping is on the device so the body can be captured in a CUDA graph."""
        c = self.cfg
        pos = self.positions
        act = self.active
        blk = torch.gather(self.block_table, 1, (pos // BLOCK_SIZE).long().clamp_(max=self.max_blocks_per_seq - 1)[:, None]).squeeze(1)
        slot_map = torch.where(act > 0, blk.long() * BLOCK_SIZE + (pos % BLOCK_SIZE).long(), torch.full_like(blk, -1, dtype=torch.int64))
        self.kv_lens.copy_(torch.where(act > 0, pos + 1, torch.zeros_like(pos)))
        scale = 1.0 / math.sqrt(c.head_dim)

        def attn(li, qkv):
            q = qkv[:, : c.q_size].contiguous()
            if self.native and c.head_dim == 128:
                return paged_decode_attention(q, self.cache[li], self.block_table, self.kv_lens, scale, self.decode_splits,
                                              self.max_model_len, self.workspace)
            from verl_b200.ops.attention import paged_decode_attention_ref

            return paged_decode_attention_ref(q, self.cache[li], self.block_table, self.kv_lens, scale)

        h = self._layer_stack(self.cur_tokens, pos if self.visual is None else pos + self.rope_delta, slot_map, attn)
        logits = ops.linear(h, self.model.output_weight)
        self._sample(logits, sp.temperature, sp.top_k, sp.top_p, self.row_ids, self.out_tok, self.out_lp)
        self._tp_sync_samples(self.out_tok, self.out_lp)
        self.cur_tokens.copy_(self.out_tok)
        self.positions.add_(act)
        self.hist_tok.index_copy_(0, self.hist_idx, self.out_tok[None])
        self.hist_lp.index_copy_(0, self.hist_idx, self.out_lp[None])
        if self._last_routed is not None:
            self.hist_routed.index_copy_(0, self.hist_idx, self._last_routed[None])
        if sp.top_logprobs > 0:
            tv, ti = self._top_head(logits, sp)
            self.hist_topi.index_copy_(0, self.hist_idx, ti[None])
            self.hist_topv.index_copy_(0, self.hist_idx, tv[None])
        self.hist_idx.add_(1).remainder_(self.sync_interval)
        if self.native:
            self.rng[1] += 1

    def _decode_step(self, sp: SamplingParams):
        if sp.top_logprobs > 0:
            self._ensure_top_hist(int(sp.top_logprobs))
        if self.record_routing and self.cfg.is_moe and getattr(self, "hist_routed", None) is None:
            # static buffer (allocated outside any graph capture): routing of the tokens fed in the un-synchronised steps
            self.hist_routed = torch.zeros(self.sync_interval, self.max_num_seqs, len(self.model.layers), self.cfg.num_experts_per_tok,
                                           dtype=torch.int16, device=self.device)
        if self.enforce_eager:
            self._decode_body(sp)
            return
        key = (sp.temperature, sp.top_k, sp.top_p, sp.top_logprobs)
        if self._graph is None or self._graph[0] != key:
            # warm-up on a side stream, then capture
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            saved = [t.clone() for t in (self.cur_tokens, self.positions, self.kv_lens, self.hist_idx, self.rng, self.hist_tok, self.hist_lp)]
            with torch.cuda.stream(s):
                self._decode_body(sp)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            _ext.check_status("rollout decode warm-up")
            g = torch.cuda.CUDAGraph()
            n0 = _ext.launch_count()
            with torch.cuda.graph(g):
                self._decode_body(sp)
            self._graph_launches = _ext.launch_count() - n0
            # warm-up and capture do not advance real state: the graph has not been replayed yet, restore the warm-up's effects
            for t, sv in zip((self.cur_tokens, self.positions, self.kv_lens, self.hist_idx, self.rng, self.hist_tok, self.hist_lp), saved):
                t.copy_(sv)
            self._graph = (key, g)
        self._graph[1].replay()
        _ext.add_graph_launches(self._graph_launches)

    # ------------------------------------------------------------------ request loop
    def _flush(self, pending: list, reqs: dict, sp: SamplingParams, eos_ids: set):
        """Read back the sampled tokens of the un-synchronised decode steps and retire finished sequences."""
        if not pending:
            return
        import time

        t_f = time.perf_counter()
        tok = self.hist_tok.cpu().numpy()
        lp = self.hist_lp.cpu().numpy()
        topi = topv = None
        if sp.top_logprobs > 0:
            topi, topv = self.hist_topi.cpu().numpy(), self.hist_topv.cpu().numpy()
        routed = self.hist_routed.cpu().numpy() if getattr(self, "hist_routed", None) is not None and self.record_routing else None
        freed = []
        for ring, ids, slots in pending:
            for sid, slot in zip(ids, slots):
                r = reqs[int(sid)]
                if r["done"]:
                    continue
                t = int(tok[ring, slot])
                r["out"].append(t)
                r["lp"].append(float(lp[ring, slot]))
                if routed is not None:
                    r.setdefault("routed", []).append(routed[ring, slot][None].copy())      # routing of the token FED at this step
                if topi is not None:
                    r.setdefault("topi", []).append(topi[ring, slot].tolist())
                    r.setdefault("topv", []).append(topv[ring, slot].tolist())
                if (not sp.ignore_eos) and t in eos_ids:
                    r["done"], r["stop"] = True, "stop"
                elif len(r["out"]) >= r["max_new"]:
                    r["done"], r["stop"] = True, "length"
                if r["done"]:
                    freed.append(slot)
                    r["num_preempted"] = self.sched.num_preempted(int(sid))
                    self.sched.finish(int(sid), self._cacheable_tokens(r))
                    self._report(r)
        pending.clear()
        if freed:
            self.active.index_fill_(0, torch.tensor(freed, dtype=torch.int64, device=self.device), 0)
        self.stats["t_flush"] += time.perf_counter() - t_f

    def _cacheable_tokens(self, r: dict):
        """Ids of the tokens whose KV a finished request leaves in the cache (everything but the last sampled token, which was
        never fed back), or None when its blocks must not be found by other requests."""
        if not self.enable_prefix_caching or r.get("mm"):
            return None
        return (r["prompt"] + r["out"])[:-1]

    @staticmethod
    def _prompt_key(p, mm):
        """Identity of a prompt for prefix sharing: the token ids, plus a digest of the images for multimodal prompts (the
        placeholder tokens of two different images are identical)."""
        if not mm or mm.get("pixel_values") is None:
            return tuple(p)
        pv = torch.as_tensor(mm["pixel_values"]).float()
        return (tuple(p), tuple(pv.shape), round(float(pv.sum()), 4), round(float(pv.abs().sum()), 4))

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sampling_params: Optional[SamplingParams] = None,
                 eos_token_id=None, admit=None, on_done=None, keep_alive=None, should_abort=None, multi_modal=None) -> list[TokenOutput]:
        """Batch generation, optionally kept open as a serving loop. ``multi_modal``: per prompt ``None`` or
        ``{"pixel_values", "image_grid_thw"}`` (the prompt then holds the expanded image placeholder tokens); ``admit`` may
        return such a dict as a third tuple element.

        With ``admit`` (a callable returning a list of ``(prompt_ids, max_tokens or None)``) new requests join the
        running batch whenever the loop synchronises with the device; they are numbered consecutively after the initial
        prompts. ``on_done(request_index, TokenOutput)`` fires as each request finishes; the loop runs while work is left
        or ``keep_alive()`` is true. ``should_abort()`` returning true ends every live request with
        ``stop_reason="aborted"`` and its partial output. All requests of one call share ``sampling_params`` except
        ``max_tokens``.
        """
        sp = sampling_params or SamplingParams()
        self.wake_up()
        eos_ids = set() if eos_token_id is None else ({eos_token_id} if isinstance(eos_token_id, int) else set(eos_token_id))
        eos_ids |= set(sp.stop_token_ids)
        self.rng[0] = sp.seed
        self._cpu_gen.manual_seed(sp.seed)
        self.active.zero_()
        reqs: dict[int, dict] = {}
        counts: dict[tuple, int] = {}
        self._on_done, self._sp_logprobs = on_done, sp.logprobs
        poll_no = 0

        def add_requests(items):
            nonlocal poll_no
            poll_no += 1
            local: dict[tuple, int] = {}
            items = [(it[0], it[1], it[2] if len(it) > 2 else None) for it in items]
            if self.enable_prefix_sharing:
                for p, _, mm in items:
                    k = self._prompt_key(p, mm)
                    local[k] = local.get(k, 0) + 1
            for p, mt, mm in items:
                i = len(reqs)
                p = list(p)
                pk = self._prompt_key(p, mm)
                max_new = min(int(mt) if mt else sp.max_tokens, self.max_model_len - len(p))
                if max_new <= 0:
                    raise ValueError(f"prompt {i} of length {len(p)} leaves no room below max_model_len={self.max_model_len}")
                key = 0
                if local.get(pk, 0) > 1:
                    key = (hash((poll_no, pk)) & 0x3FFFFFFFFFFFFFFF) or 1
                    counts[pk] = local[pk]
                reqs[i] = {"id": i, "prompt": p, "out": [], "lp": [], "done": False, "stop": None, "max_new": max_new, "n_gen": 0,
                           "num_preempted": 0, "slot": -1, "reported": False, "pkey": pk}
                if mm:
                    assert self.visual is not None, "this engine was built without a vision tower"
                    from verl_b200.models.vision import get_rope_index

                    reqs[i]["mm"] = mm
                    reqs[i]["rope_delta"] = get_rope_index(torch.as_tensor(p), mm.get("image_grid_thw"), self.vision_config, grid_t_scale=mm.get("grid_t_scale"))[1]
                self.sched.add(i, len(p), max_new, key, tokens=p, no_chunk=bool(mm), no_cache=bool(mm))

        add_requests([(p, None, multi_modal[j] if multi_modal is not None else None) for j, p in enumerate(prompts)])
        owner_logits: dict[int, torch.Tensor] = {}
        owner_routed: dict[int, np.ndarray] = {}
        owner_partial_block: dict[int, int] = {}
        pending: list = []
        ring = int(self.hist_idx.item())
        n_preempt = self.sched.num_preemptions
        while True:
            if not pending:     # the host is in sync with the device here: a safe point to change the request set
                if should_abort is not None and should_abort():
                    for r in reqs.values():
                        if not r["done"]:
                            r["done"], r["stop"] = True, "aborted"
                            self._report(r)
                    self.sched.abort_all()
                    self.active.zero_()
                    break
                if admit is not None:
                    fresh_items = admit()
                    if fresh_items:
                        add_requests(fresh_items)
            kind, ids, slots, lens, forks = self.sched.step()
            if kind == STEP_IDLE:
                self._flush(pending, reqs, sp, eos_ids)
                if self.sched.num_running == 0 and self.sched.num_waiting == 0:
                    if keep_alive is not None and keep_alive():
                        time.sleep(0.001)
                        continue
                    break
                if all(r["done"] for r in reqs.values()) and not (keep_alive is not None and keep_alive()):
                    break
                continue
            if kind == STEP_PREFILL:
                self._flush(pending, reqs, sp, eos_ids)
                ids, slots, forks, lens, starts = ids.copy(), slots.copy(), forks.copy(), lens.copy(), self.sched.starts.copy()
                fresh = [(reqs[int(s)], int(sl), int(st), int(n)) for s, sl, f, st, n in zip(ids, slots, forks, starts, lens)
                         if f < 0 and not reqs[int(s)]["done"]]
                forked = [(reqs[int(s)], int(sl), int(f)) for s, sl, f in zip(ids, slots, forks) if f >= 0]
                for s in ids:  # a sequence that finished while waiting for re-admission
                    if reqs[int(s)]["done"]:
                        self.sched.finish(int(s))
                t_pf = self._tick()
                started = []
                if fresh:
                    logits, fin = self._prefill(fresh, sp)
                    started = [(fresh[i][0], fresh[i][1]) for i in fin]      # the others have more prompt chunks to go
                    for row, (r, sl) in enumerate(started):
                        r["slot"] = sl
                        if counts.get(r["pkey"], 0) > 1 and not r["out"]:
                            owner_logits[r["id"]] = logits[row]
                            if "routed" in r:
                                owner_routed[r["id"]] = np.concatenate(r["routed"], 0)
                            owner_partial_block[r["id"]] = int(self.block_table_host[sl, len(r["prompt"]) // BLOCK_SIZE])
                    if started:
                        self._start_sequences(started, logits, sp)
                if forked:
                    src_b, dst_b, rows = [], [], []
                    for r, slot, owner in forked:
                        blocks = self.sched.blocks(r["id"])
                        self.block_table_host[slot, : len(blocks)] = blocks
                        self.block_table_host[slot, len(blocks):] = 0
                        P = len(r["prompt"])
                        if P % BLOCK_SIZE:
                            src_b.append(owner_partial_block[owner])
                            dst_b.append(int(blocks[P // BLOCK_SIZE]))
                        rows.append(owner_logits[owner])
                        if owner in owner_routed:
                            r["routed"] = [owner_routed[owner]]
                    if src_b:
                        si = torch.tensor(src_b, device=self.device)
                        di = torch.tensor(dst_b, device=self.device)
                        self.cache[:, di] = self.cache[:, si]
                    self._start_sequences([(r, s) for r, s, _ in forked], torch.stack(rows), sp)
                    self.stats["forked"] += len(forked)
                for r, sl, *_ in fresh:
                    r["slot"] = sl
                for r, sl, _ in forked:
                    r["slot"] = sl
                self._push_block_table()
                # sequences whose single allowed token came from the prefill are complete
                done_now = [(r, sl) for r, sl in started + [(r, s) for r, s, _ in forked]
                            if len(r["out"]) >= r["max_new"] or ((not sp.ignore_eos) and r["out"][-1] in eos_ids)]
                for r, sl in done_now:
                    r["done"], r["stop"] = True, ("length" if len(r["out"]) >= r["max_new"] else "stop")
                    self.sched.finish(r["id"], self._cacheable_tokens(r))
                    self.active[sl] = 0
                    self._report(r)
                self.stats["t_prefill"] += self._tick() - t_pf
                continue
            # ---- decode
            ids, slots, lens = ids.copy(), slots.copy(), lens.copy()
            if self.sched.num_preemptions != n_preempt:
                n_preempt = self.sched.num_preemptions
                self.stats["preemptions"] = n_preempt
                self._flush(pending, reqs, sp, eos_ids)
                self.active.zero_()
                live = [int(sl) for s, sl in zip(ids, slots) if not reqs[int(s)]["done"]]
                if live:
                    self.active.index_fill_(0, torch.tensor(live, dtype=torch.int64, device=self.device), 1)
            grew = np.nonzero((lens - 1) % BLOCK_SIZE == 0)[0]   # these sequences write the first slot of a new block
            for j in grew:
                blocks = self.sched.blocks(int(ids[j]))
                self.block_table_host[slots[j], : len(blocks)] = blocks
            if len(grew):
                self._push_block_table()
            if self._graph is None and not self.enforce_eager:
                t_c = self._tick()
                self._decode_step(sp)
                self.stats["t_capture"] += self._tick() - t_c
            else:
                self._decode_step(sp)
            self.stats["decode_steps"] += 1
            pending.append((ring, ids, slots))
            ring = (ring + 1) % self.sync_interval
            at_limit = False
            for s in ids.tolist():
                r = reqs[s]
                r["n_gen"] += 1
                if r["n_gen"] >= r["max_new"] and not r["done"]:
                    at_limit = True
            if at_limit or len(pending) >= self.sync_interval:
                self._flush(pending, reqs, sp, eos_ids)
        if self.native:
            _ext.check_status("rollout generate")
        if self.sched is not None:
            hit, chunks = self.sched.prefix_cache_hit_tokens, self.sched.extra_prefill_chunks
            self.stats["prefix_cache_hit_tokens"] += hit - self._sched_counted[0]
            self.stats["prefill_chunks"] += chunks - self._sched_counted[1]
            self._sched_counted = [hit, chunks]
        outs = []
        for i in range(len(prompts)):
            r = reqs[i]
            outs.append(TokenOutput(token_ids=r["out"][: r["max_new"]], log_probs=r["lp"][: r["max_new"]] if sp.logprobs else None,
                                    top_ids=r["topi"][: r["max_new"]] if "topi" in r else None,
                                    top_log_probs=r["topv"][: r["max_new"]] if "topv" in r else None, routed_experts=self._routed_of(r),
                                    stop_reason=r["stop"] or "length", num_preempted=r["num_preempted"]))
        return outs

    @staticmethod
    def _routed_of(r: dict) -> Optional[np.ndarray]:
        """[prompt + response, layers, topk] int16: the experts chosen for every token of the sequence. The last sampled token
        is never fed to the model, so its row repeats the previous one (the trainer does not use that position's output)."""
        if not r.get("routed"):
            return None
        n_out = len(r["out"][: r["max_new"]])
        want = len(r["prompt"]) + n_out
        rt = np.concatenate(r["routed"], 0)[:want]
        if rt.shape[0] < want:
            rt = np.concatenate([rt, np.repeat(rt[-1:], want - rt.shape[0], 0)], 0)
        return rt

    def _report(self, r: dict):
        if r.get("reported") or getattr(self, "_on_done", None) is None:
            return
        r["reported"] = True
        self._on_done(r["id"], TokenOutput(token_ids=r["out"][: r["max_new"]], log_probs=r["lp"][: r["max_new"]] if self._sp_logprobs else None,
                                           top_ids=r["topi"][: r["max_new"]] if "topi" in r else None,
                                           top_log_probs=r["topv"][: r["max_new"]] if "topv" in r else None, routed_experts=self._routed_of(r),
                                           stop_reason=r["stop"] or "length", num_preempted=r["num_preempted"]))

    @torch.no_grad()
    def score_prompts(self, prompts: Sequence[Sequence[int]], k: int, max_tokens_per_pass: int = 16384, chunk: int = 2048) -> list:
        """Forward-only scoring of whole sequences (no sampling, no KV cache): for every sequence ``(ids [L, max(k, 1)] int32,
        log_probs [L, max(k, 1)] float32)``. Row i describes the distribution for token i given tokens < i: with ``k > 0`` its k most
        likely tokens and their log-probs, with ``k == 0`` the token that is there and its log-prob. Row 0 has no context: it
        holds the token itself with log-prob 0. Sequences are packed into passes of at most ``max_tokens_per_pass`` tokens and the
        vocabulary projection runs over ``chunk`` rows at a time, so no [L, V] tensor outlives its chunk."""
        from verl_b200.models.transformer import PackedBatch

        if getattr(self, "tp_size", 1) > 1:
            raise NotImplementedError("prompt scoring runs on tensor_model_parallel_size=1 replicas")
        model, dev = self.model, self.device
        W = model.output_weight
        kk = max(int(k), 1)
        out = [None] * len(prompts)
        order = sorted(range(len(prompts)), key=lambda i: len(prompts[i]))
        i = 0
        while i < len(order):
            group, tot = [], 0
            while i < len(order) and (not group or tot + len(prompts[order[i]]) <= max_tokens_per_pass):
                group.append(order[i])
                tot += len(prompts[order[i]])
                i += 1
            lens = [len(prompts[j]) for j in group]
            ids = torch.tensor([t for j in group for t in prompts[j]], dtype=torch.long, device=dev)
            pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).to(dev)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
            h = model.forward_hidden(PackedBatch(ids, pos, cu.to(dev), cu, max(lens)))
            top_i = torch.empty(tot, kk, dtype=torch.int32, device=dev)
            top_l = torch.empty(tot, kk, dtype=torch.float32, device=dev)
            nxt_all = torch.cat([ids[1:], ids.new_zeros(1)])
            for a in range(0, tot, chunk):
                lp = torch.log_softmax(torch.nn.functional.linear(h[a:a + chunk], W).float(), -1)
                if k > 0:
                    v, ix = lp.topk(kk, dim=-1)
                else:      # the log-prob of the NEXT token in the stream (shifted into place below; a sequence's last row is dropped)
                    nxt = nxt_all[a:a + chunk]
                    ix, v = nxt[:, None], lp.gather(-1, nxt[:, None])
                top_i[a:a + lp.shape[0]], top_l[a:a + lp.shape[0]] = ix.to(torch.int32), v
            top_i, top_l = top_i.cpu(), top_l.cpu()
            off = 0
            for j, n in zip(group, lens):
                oi = torch.empty(n, kk, dtype=torch.int32)
                ol = torch.zeros(n, kk, dtype=torch.float32)
                oi[0] = int(prompts[j][0])
                oi[1:], ol[1:] = top_i[off:off + n - 1], top_l[off:off + n - 1]         # the prediction made at row i-1 describes token i
                out[j] = (oi, ol)
                off += n
        return out

    def abort_all(self) -> list[int]:
        """Drop every live request (used when a weight update interrupts generation)."""
        ids = self.sched.abort_all() if self.sched is not None else []
        if hasattr(self, "active"):
            self.active.zero_()
        return ids
