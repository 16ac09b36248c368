"""Decoder-only transformer (Llama / Qwen2 / Qwen3 / Qwen3-MoE families) on packed variable-length batches.

The model is written against ``verl_b200.ops`` so the same definition runs the sm_100a kernels on a B200 and plain
PyTorch on CPU. Inputs are *packed*: all sequences of a micro-batch back to back in one ``[T]`` row with
``cu_seqlens`` marking the boundaries (what the reference obtains by monkey-patching HF models for
``use_remove_padding``: ``verl/models/transformers/monkey_patch.py:87-156``,
``verl/workers/engine/fsdp/transformer_impl.py:1155-1342``). Projections are stored fused (``qkv_proj``,
``gate_up_proj``) and converted from/to HF tensor names on import/export.
"""

from __future__ import annotations

import math
from typing import Iterator, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from verl_b200 import ops
from verl_b200.models.config import ModelConfig
from verl_b200.parallel.tp import (allgather_linear, copy_to_tp, gather_from_sp, linear_reduce_scatter, reduce_from_tp, reduce_scatter_to_sp,
                                  vocab_parallel_embedding)

__all__ = ["DecoderLM", "PackedBatch", "hf_to_native_state_dict", "native_to_hf_tensors"]


class PackedBatch:
    """Device-side description of a packed micro-batch."""

    __slots__ = ("input_ids", "position_ids", "cu_seqlens", "cu_seqlens_cpu", "max_seqlen", "routed_experts", "global_position_ids",
                 "attn_expand", "visual_embeds", "visual_token_ids", "rope_override", "mm", "cp_zigzag", "deepstack_embeds", "visual_rows")

    def __init__(self, input_ids, position_ids, cu_seqlens, cu_seqlens_cpu=None, max_seqlen=None, routed_experts=None):
        self.input_ids = input_ids
        self.position_ids = position_ids
        self.cu_seqlens = cu_seqlens.to(torch.int32)
        self.cu_seqlens_cpu = cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu()
        lens = self.cu_seqlens_cpu[1:] - self.cu_seqlens_cpu[:-1]
        self.max_seqlen = int(max_seqlen if max_seqlen is not None else (lens.max() if lens.numel() else 0))
        self.routed_experts = routed_experts  # optional [T, layers, topk] forced routing (router replay)
        # sequence parallelism: input_ids / position_ids are this rank's slice, cu_seqlens describe the whole micro-batch and
        # this holds the (padded) positions of all its tokens
        self.global_position_ids = None
        # prefix sharing: (expand [E], back [T], order [E], offsets [T + 1]) int64 index tensors. input_ids / position_ids then hold every distinct prompt
        # once; cu_seqlens describe the E-row layout of full sequences that attention runs on (rows = x[expand]) and
        # back picks, for each of the T stored tokens, its row of that layout (see verl_b200.utils.prefix_sharing)
        self.attn_expand = None
        # vision-language models (verl_b200.models.vision): rows that replace the embeddings of the image placeholder tokens,
        # and per-token rotary tables (cos, sin) [T, D/2] of the multimodal rotary embedding
        self.visual_embeds = self.visual_token_ids = self.rope_override = self.mm = None
        # deep-stack vision features (Qwen3-VL): entry i [n_visual_tokens, H] is added to the stream at the visual rows after decoder
        # layer i; visual_rows caches the indices of those rows
        self.deepstack_embeds = self.visual_rows = None
        self.cp_zigzag = False        # context parallelism: the local rows are two chunks of the stream (zig-zag placement)


def _proj(mod: nn.Module, name: str, x: torch.Tensor, bias=None) -> torch.Tensor:
    """``x @ Wᵀ (+ bias)`` plus the low-rank update ``scale · (x Aᵀ) Bᵀ`` when the module carries a LoRA adapter for ``name``
    (see ``verl_b200.models.lora``)."""
    w = getattr(mod, name)
    if getattr(w, "_zero3", None) is not None:      # row-sharded weight of the ZeRO-3 engine: gather fused into the GEMM
        from verl_b200.workers.engine.fsdp.zero3 import zero3_linear

        return zero3_linear(x, w, bias)
    y = ops.linear(x, w, bias)
    adapters = getattr(mod, "_lora", None)
    if adapters and name in adapters:
        a, b, scale = adapters[name]
        y = y + ops.linear(ops.linear(x, getattr(mod, a)), getattr(mod, b)) * scale
    return y


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        self.qkv_proj = nn.Parameter(torch.empty(cfg.q_size + 2 * cfg.kv_size, cfg.hidden_size, **kw))
        self.qkv_bias = nn.Parameter(torch.zeros(cfg.q_size + 2 * cfg.kv_size, **kw)) if cfg.attention_bias else None
        self.o_proj = nn.Parameter(torch.empty(cfg.hidden_size, cfg.q_size, **kw))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw))
        self.tp_group = None    # set by the tensor-parallel engine; cfg then describes the LOCAL head counts

    def forward(self, x: torch.Tensor, pb: PackedBatch, cos, sin, sp_group=None) -> torch.Tensor:
        cfg = self.cfg
        fu = getattr(self, "fused_ulysses", None)
        if sp_group is not None and fu is not None and not cfg.qk_norm and not getattr(self, "_lora", None) and pb.global_position_ids is not None:
            from verl_b200.parallel.ulysses import fused_ulysses_attention_block

            return fused_ulysses_attention_block(x, self, pb, cfg, fu, cos, sin)
        if getattr(self, "tp_sp", False):       # sequence-parallel region boundary: all-gather fused into the projection
            qkv = allgather_linear(x, self.qkv_proj, self.qkv_bias, self.tp_group, getattr(self, "tp_ctx", None))
        else:
            qkv = _proj(self, "qkv_proj", copy_to_tp(x, self.tp_group), self.qkv_bias)
        if cfg.qk_norm:
            T = qkv.shape[0]
            q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=-1)
            q = ops.rmsnorm(q.reshape(-1, cfg.head_dim), self.q_norm, cfg.rms_norm_eps).reshape(T, cfg.q_size)
            k = ops.rmsnorm(k.reshape(-1, cfg.head_dim), self.k_norm, cfg.rms_norm_eps).reshape(T, cfg.kv_size)
            qkv = torch.cat([q, k, v], dim=-1)
        qkv = ops.apply_rope_(qkv, pb.position_ids, cos, sin, cfg.num_attention_heads + cfg.num_key_value_heads, cfg.head_dim)
        if sp_group is not None and getattr(self, "sp_mode", "ulysses") == "context":
            from verl_b200.parallel.context_parallel import context_parallel_attention

            o = context_parallel_attention(qkv, pb, cfg, sp_group)     # all-gather K/V, attention for the local query rows
        elif sp_group is not None:
            from verl_b200.parallel.ulysses import ulysses_attention

            o = ulysses_attention(qkv, pb, cfg, sp_group)
        elif pb.attn_expand is not None:
            from verl_b200.utils.prefix_sharing import expand_rows, select_rows

            expand, back, order, offsets = pb.attn_expand
            o = select_rows(ops.attention_varlen(expand_rows(qkv, expand, order, offsets), pb.cu_seqlens, cfg.num_attention_heads,
                                                 cfg.num_key_value_heads, cfg.head_dim, pb.max_seqlen, pb.cu_seqlens_cpu), back)
        else:
            o = ops.attention_varlen(qkv, pb.cu_seqlens, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                     pb.max_seqlen, pb.cu_seqlens_cpu)
        if getattr(self, "tp_sp", False):
            return linear_reduce_scatter(o, self.o_proj, self.tp_group, getattr(self, "tp_ctx", None))
        return reduce_from_tp(_proj(self, "o_proj", o), self.tp_group)


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.xielu = getattr(cfg, "mlp_act", "swiglu") == "xielu"
        if self.xielu:
            # Apertus: no gate; the activation's two curvature parameters are learned per layer (stored before their softplus)
            self.up_proj = nn.Parameter(torch.empty(cfg.intermediate_size, cfg.hidden_size, **kw))
            self.act_alpha_p = nn.Parameter(torch.empty(1, **kw))
            self.act_alpha_n = nn.Parameter(torch.empty(1, **kw))
        else:
            self.gate_up_proj = nn.Parameter(torch.empty(2 * cfg.intermediate_size, cfg.hidden_size, **kw))
        self.down_proj = nn.Parameter(torch.empty(cfg.hidden_size, cfg.intermediate_size, **kw))
        self.tp_group = None

        self.tiled_shards = 0          # > 1: token-tiled execution with per-tile recomputation in backward (``_TiledMLP``)

    def forward(self, x):
        if self.tiled_shards > 1 and not getattr(self, "tp_sp", False) and x.shape[0] >= 2 * self.tiled_shards:
            return _TiledMLP.apply(x, self, self.tiled_shards, *[p for p in self.parameters() if p.requires_grad])
        return self._dense(x)

    XIELU_BETA, XIELU_EPS = 0.5, -1e-6

    def _xielu(self, u):
        """xIELU (arXiv 2411.13010): alpha_p x^2 + beta x for x > 0, alpha_n (expm1(min(x, eps)) - x) + beta x otherwise."""
        ap = F.softplus(self.act_alpha_p.float())
        an = self.XIELU_BETA + F.softplus(self.act_alpha_n.float())
        x = u.float()
        y = torch.where(x > 0, ap * x * x + self.XIELU_BETA * x, (torch.expm1(torch.clamp(x, max=self.XIELU_EPS)) - x) * an + self.XIELU_BETA * x)
        return y.to(u.dtype)

    def _dense(self, x):
        if self.xielu:
            if getattr(self, "tp_sp", False):
                tpctx = getattr(self, "tp_ctx", None)
                return linear_reduce_scatter(self._xielu(allgather_linear(x, self.up_proj, None, self.tp_group, tpctx)), self.down_proj, self.tp_group, tpctx)
            y = _proj(self, "down_proj", self._xielu(_proj(self, "up_proj", copy_to_tp(x, self.tp_group))))
            return reduce_from_tp(y, self.tp_group)
        if getattr(self, "tp_sp", False):
            tpctx = getattr(self, "tp_ctx", None)
            h = ops.swiglu(allgather_linear(x, self.gate_up_proj, None, self.tp_group, tpctx))
            return linear_reduce_scatter(h, self.down_proj, self.tp_group, tpctx)
        y = _proj(self, "down_proj", ops.swiglu(_proj(self, "gate_up_proj", copy_to_tp(x, self.tp_group))))
        return reduce_from_tp(y, self.tp_group)


class _TiledMLP(torch.autograd.Function):
    """The MLP over ``shards`` slices of the token axis. Forward keeps nothing but the input: the [T, 2I] gate/up activations
    and the [T, I] product exist for one slice at a time. Backward recomputes each slice and back-propagates through it; the
    weight gradients of the slices add up in ``main_grad`` (fp32, inside the weight-gradient GEMM) or in ``.grad``.
    Reference: ``verl/models/transformers/tiled_mlp.py:86-229`` (``TiledMLP`` with a gradient accumulator for FSDP); the
    parameters are passed as inputs only so that autograd calls this node when they need gradients."""

    @staticmethod
    def forward(ctx, x, mlp, shards, *params):
        ctx.mlp, ctx.shards = mlp, shards
        ctx.save_for_backward(x)
        bounds = _tile_bounds(x.shape[0], shards)
        with torch.no_grad():
            return torch.cat([mlp._dense(x[a:b]) for a, b in bounds], 0)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        mlp = ctx.mlp
        params = [p for p in mlp.parameters() if p.requires_grad]
        dx = torch.empty_like(x)
        acc = [None] * len(params)
        for a, b in _tile_bounds(x.shape[0], ctx.shards):
            xs = x[a:b].detach().requires_grad_(True)
            with torch.enable_grad():
                ys = mlp._dense(xs)
            grads = torch.autograd.grad(ys, [xs] + params, dy[a:b], allow_unused=True)
            dx[a:b] = grads[0]
            for i, g in enumerate(grads[1:]):       # None when the projection accumulated into main_grad itself
                if g is not None:
                    acc[i] = g if acc[i] is None else acc[i] + g
        return (dx, None, None, *acc)


def _tile_bounds(T: int, shards: int):
    """Token slices of near-equal size, each a multiple of 128 rows where the length allows (full GEMM tiles)."""
    per = -(-T // shards)
    if T >= 256 * shards:
        per = -(-per // 128) * 128
    return [(a, min(T, a + per)) for a in range(0, T, per)]


class MoE(nn.Module):
    """Top-k softmax-routed experts (Qwen3-MoE). Experts are stored packed [E, 2I, H] / [E, H, I]; the token
    permutation + grouped GEMM path lives in ``verl_b200.ops.moe``; expert parallelism in ``verl_b200.parallel.ep``."""

    def __init__(self, cfg: ModelConfig, dtype, device, layer_idx: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        kw = dict(dtype=dtype, device=device)
        E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
        self.router = nn.Parameter(torch.empty(E, H, **kw))
        self.experts_gate_up = nn.Parameter(torch.empty(E, 2 * I, H, **kw))
        self.experts_down = nn.Parameter(torch.empty(E, H, I, **kw))
        self.ep_group = None
        self.ep_ctx = None      # FusedEPContext: dispatch / combine run inside the grouped GEMMs over peer memory
        self.tp_group = None    # expert tensor parallelism: every expert's intermediate dimension is split
        self.last_topk: Optional[torch.Tensor] = None   # recorded routing (router replay R2)
        self.record_routing = False

    def forward(self, x, forced_topk: Optional[torch.Tensor] = None):
        from verl_b200.ops.moe import moe_forward

        out, topk_idx = moe_forward(copy_to_tp(x, self.tp_group), self.router, self.experts_gate_up, self.experts_down,
                                    self.cfg.num_experts_per_tok, self.cfg.norm_topk_prob, forced_topk=forced_topk, ep_group=self.ep_group,
                                    ep_ctx=self.ep_ctx)
        if self.record_routing:
            self.last_topk = topk_idx.detach()
        return reduce_from_tp(out, self.tp_group)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, layer_idx: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        kw = dict(dtype=dtype, device=device)
        self.input_layernorm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        self.post_attention_layernorm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        self.self_attn = Attention(cfg, dtype, device)
        self.mlp = MoE(cfg, dtype, device, layer_idx) if cfg.is_moe else MLP(cfg, dtype, device)

    def forward(self, h, residual, pb: PackedBatch, cos, sin, sp_group=None):
        """(h, residual) carry the un-normalised stream split in two so the add is fused into the next norm."""
        if residual is None:
            residual = h
            x = ops.rmsnorm(h, self.input_layernorm, self.cfg.rms_norm_eps)
        else:
            x, residual = ops.add_rmsnorm(h, residual, self.input_layernorm, self.cfg.rms_norm_eps)
        a = self.self_attn(x, pb, cos, sin, sp_group)
        x, residual = ops.add_rmsnorm(a, residual, self.post_attention_layernorm, self.cfg.rms_norm_eps)
        if self.cfg.is_moe:
            forced = pb.routed_experts[:, self.layer_idx] if pb.routed_experts is not None else None
            m = self.mlp(x, forced)
        else:
            m = self.mlp(x)
        return m, residual


class DecoderLM(nn.Module):
    """Embedding → N decoder layers → final norm → (lm_head | value head)."""

    def __init__(self, cfg: ModelConfig, dtype: torch.dtype = torch.bfloat16, device="cpu", init: bool = True, seed: int = 0,
                 layer_range: Optional[range] = None, pre_process: bool = True, post_process: bool = True):
        """``layer_range`` / ``pre_process`` / ``post_process`` build one pipeline stage: only those decoder layers, the
        embedding only on the first stage, final norm and head only on the last. Local layer j is global layer
        ``layer_range.start + j``."""
        super().__init__()
        self.cfg = cfg
        self.dtype = dtype
        kw = dict(dtype=dtype, device=device)
        layer_range = range(cfg.num_hidden_layers) if layer_range is None else layer_range
        self.layer_offset, self.pre_process, self.post_process = layer_range.start, pre_process, post_process
        self.tp_group, self.vocab_offset = None, 0
        self.gradient_checkpointing = False
        self.sp_group = None
        self.layers = nn.ModuleList([DecoderLayer(cfg, dtype, device, i) for i in layer_range])
        if pre_process or (post_process and cfg.tie_word_embeddings and not cfg.value_head):
            self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.lm_head = None
        if not post_process:
            if init:
                self.reset_parameters(seed)
            return
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        if cfg.value_head:
            self.score = nn.Parameter(torch.empty(1, cfg.hidden_size, **kw))
            self.lm_head = None
        elif cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        if init:
            self.reset_parameters(seed)

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def reset_parameters(self, seed: int = 0):
        """normal(0, initializer_range) for matrices, ones for norms, zeros for biases (HF ``_init_weights``)."""
        gen = torch.Generator(device=next(self.parameters()).device)
        gen.manual_seed(seed)
        std = self.cfg.initializer_range
        for name, p in self.named_parameters():
            if name.endswith("layernorm") or name.endswith("norm"):
                p.fill_(1.0)
            elif name.endswith("bias"):
                p.zero_()
            elif name.endswith("act_alpha_p"):
                p.fill_(math.log(math.expm1(0.8)))              # softplus^-1 of the published start values (0.8, and 0.8 - beta)
            elif name.endswith("act_alpha_n"):
                p.fill_(math.log(math.expm1(0.8 - MLP.XIELU_BETA)))
            else:
                p.normal_(0.0, std, generator=gen)

    @property
    def output_weight(self) -> torch.Tensor:
        return self.embed_tokens if self.lm_head is None else self.lm_head

    # ------------------------------------------------------------------ forward
    def rope(self, device):
        return ops.rope_tables(self.cfg.max_position_embeddings, self.cfg.head_dim, self.cfg.rope_theta, device, self.cfg.rope_scaling)

    def set_tp_group(self, group, vocab_offset: int = 0, sequence_parallel: bool = False, tp_ctx=None):
        """Switch the model to tensor-parallel execution: ``cfg`` must already describe the local shard. With
        ``sequence_parallel`` the stream between the attention / MLP blocks is split over tokens (``[T/tp, H]`` per rank)."""
        self.tp_group, self.vocab_offset, self.tp_sp = group, vocab_offset, sequence_parallel
        for layer in self.layers:
            for mod in (layer.self_attn, layer.mlp):
                mod.tp_group, mod.tp_sp, mod.tp_ctx = group, sequence_parallel, tp_ctx

    def forward_hidden(self, pb: PackedBatch, h_in: Optional[torch.Tensor] = None):
        """Final-normed hidden states [T, H] on the last pipeline stage, the raw residual stream on earlier stages.
        ``h_in`` is the stream received from the previous stage (stages without the embedding)."""
        if getattr(self.cfg, "sliding_window", 0) and pb.max_seqlen > self.cfg.sliding_window:
            raise NotImplementedError(f"this checkpoint uses sliding-window attention over {self.cfg.sliding_window} tokens; a sequence of "
                                      f"{pb.max_seqlen} tokens would need windowed attention kernels, which are not built (full attention is exact "
                                      "only up to the window)")
        cos, sin = self.rope(pb.input_ids.device)
        if pb.rope_override is not None:
            # multimodal rotary embedding: the tables already hold one row per token, so the rotary kernel indexes them by row
            cos, sin = pb.rope_override
            pb.position_ids = torch.arange(pb.input_ids.shape[0], dtype=torch.int32, device=pb.input_ids.device)
        sp = getattr(self, "tp_sp", False)
        if self.pre_process:
            if self.tp_group is not None and sp:
                h = vocab_parallel_embedding(pb.input_ids, self.embed_tokens, self.vocab_offset, None)    # partial sums
                h = reduce_scatter_to_sp(h, self.tp_group)
            elif self.tp_group is not None:
                h = vocab_parallel_embedding(pb.input_ids, self.embed_tokens, self.vocab_offset, self.tp_group)
            else:
                h = ops.embedding(pb.input_ids, self.embed_tokens)
            if pb.visual_embeds is not None:
                is_vis = torch.isin(pb.input_ids, torch.tensor(pb.visual_token_ids, device=pb.input_ids.device))
                pb.visual_rows = is_vis.nonzero(as_tuple=True)[0]
                h = h.index_put((pb.visual_rows,), pb.visual_embeds.to(h.dtype))
        else:
            h = h_in
        residual = None
        deep = pb.deepstack_embeds if self.pre_process else None
        for li, layer in enumerate(self.layers):
            if self.gradient_checkpointing and torch.is_grad_enabled():
                h, residual = checkpoint(layer, h, residual, pb, cos, sin, self.sp_group, use_reentrant=False)
            else:
                h, residual = layer(h, residual, pb, cos, sin, self.sp_group)
            if deep is not None and li < len(deep) and pb.visual_rows is not None:
                # the stream after a layer is h + residual: adding to either term adds to the stream
                h = h.index_add(0, pb.visual_rows, deep[li].to(h.dtype))
        if not self.post_process:
            return h + residual if residual is not None else h
        if residual is None:
            out = ops.rmsnorm(h, self.norm, self.cfg.rms_norm_eps)
        else:
            out = ops.add_rmsnorm(h, residual, self.norm, self.cfg.rms_norm_eps)[0]
        return gather_from_sp(out, self.tp_group, replicated_grad=True) if sp else out

    def forward(self, pb: PackedBatch, labels: Optional[torch.Tensor] = None, temperature: float = 1.0,
                need_entropy: bool = True, return_logits: bool = False):
        """Training/inference forward on a packed batch.

        * value-head models return ``{"values": [T]}``;
        * with ``labels`` returns ``{"log_probs": [T], "entropy": [T] or None}`` through the fused lm_head kernel;
        * with ``return_logits`` returns ``{"logits": [T, V]}`` (debug / sampling on CPU).
        """
        h = self.forward_hidden(pb)
        if self.cfg.value_head:
            return {"values": F.linear(h, self.score).squeeze(-1).float()}
        out = {}
        if labels is not None:
            lp, ent = ops.linear_logprob_entropy(h, self.output_weight, labels, temperature, need_entropy)
            out["log_probs"], out["entropy"] = lp, ent
        if return_logits:
            out["logits"] = F.linear(h, self.output_weight)
        out["hidden"] = h
        return out

    # ------------------------------------------------------------------ (de)serialisation with HF names
    def hf_named_tensors(self) -> Iterator[tuple[str, torch.Tensor]]:
        return native_to_hf_tensors(self.cfg, dict(self.named_parameters()))

    def load_hf_state_dict(self, sd: dict, strict: bool = True):
        native = hf_to_native_state_dict(self.cfg, sd)
        own = dict(self.named_parameters())
        missing = [k for k in own if k not in native]
        if strict and missing:
            raise KeyError(f"missing tensors for {missing[:5]} ...")
        with torch.no_grad():
            for k, v in native.items():
                if k in own:
                    own[k].copy_(v.to(own[k].dtype))


    @torch.no_grad()
    def load_hf_stream(self, named_tensors) -> int:
        """Consume (hf_name, tensor) pairs in model order, fusing and copying one decoder layer at a time so that at most
        one layer's worth of source tensors is alive (weight hand-off from a model-parallel trainer to a rollout copy).
        Returns the number of native parameters written."""
        own = dict(self.named_parameters())
        written = 0

        def flush(group: dict):
            nonlocal written
            for k, v in hf_to_native_state_dict(self.cfg, group).items():
                if k in own:
                    own[k].copy_(v.to(own[k].dtype))
                    written += 1

        group, key = {}, None
        for name, t in named_tensors:
            parts = name.split(".")
            k = ".".join(parts[:3]) if name.startswith("model.layers.") else name
            if key is not None and k != key and group:
                flush(group)
                group = {}
            key = k
            group[name] = t
        if group:
            flush(group)
        return written


# ---------------------------------------------------------------------------------------------------- name mapping
def native_to_hf_tensors(cfg: ModelConfig, params: dict) -> Iterator[tuple[str, torch.Tensor]]:
    """Yield (hf_name, tensor) splitting the fused projections; tensors are views where possible. Parameters of a
    vision-language model (``language_model.*`` + ``visual.*``) are accepted too: the tower's names pass through."""
    if any(k.startswith("language_model.") for k in params.keys()):
        class _Sub:
            """The decoder's entries under their own names; values are read through ``params[...]`` one at a time (a mapping
            that gathers sharded tensors on access keeps doing so)."""

            def __contains__(self, k):
                return "language_model." + k in params

            def __getitem__(self, k):
                return params["language_model." + k]

            def get(self, k, default=None):
                return self[k] if k in self else default

            def keys(self):
                return [k[len("language_model."):] for k in params.keys() if k.startswith("language_model.")]

        yield from native_to_hf_tensors(cfg, _Sub())
        v = cfg.vision or {}
        for k in list(params.keys()):
            if k.startswith("visual."):
                t = params[k]
                if k == "visual.patch_embed.proj.weight" and v and t.dim() == 2:
                    t = t.view(t.shape[0], v["in_channels"], v["temporal_patch_size"], v["patch_size"], v["patch_size"])
                yield ("model." + k if v.get("variant") == "qwen3_vl" else k), t
        return
    if "embed_tokens" in params:
        yield "model.embed_tokens.weight", params["embed_tokens"]
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        hp = f"model.layers.{i}."
        if p + "input_layernorm" not in params:
            continue  # pipeline stage that does not own this layer
        apertus = getattr(cfg, "mlp_act", "swiglu") == "xielu"
        yield hp + ("attention_layernorm.weight" if apertus else "input_layernorm.weight"), params[p + "input_layernorm"]
        yield hp + ("feedforward_layernorm.weight" if apertus else "post_attention_layernorm.weight"), params[p + "post_attention_layernorm"]
        qkv = params[p + "self_attn.qkv_proj"]
        q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
        yield hp + "self_attn.q_proj.weight", q
        yield hp + "self_attn.k_proj.weight", k
        yield hp + "self_attn.v_proj.weight", v
        if cfg.attention_bias:
            qb, kb, vb = params[p + "self_attn.qkv_bias"].split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
            yield hp + "self_attn.q_proj.bias", qb
            yield hp + "self_attn.k_proj.bias", kb
            yield hp + "self_attn.v_proj.bias", vb
        yield hp + "self_attn.o_proj.weight", params[p + "self_attn.o_proj"]
        if cfg.qk_norm:
            yield hp + "self_attn.q_norm.weight", params[p + "self_attn.q_norm"]
            yield hp + "self_attn.k_norm.weight", params[p + "self_attn.k_norm"]
        if cfg.is_moe:
            yield hp + "mlp.gate.weight", params[p + "mlp.router"]
            gu, dn = params[p + "mlp.experts_gate_up"], params[p + "mlp.experts_down"]
            I = cfg.moe_intermediate_size
            for e in range(cfg.num_experts):
                yield hp + f"mlp.experts.{e}.gate_proj.weight", gu[e, :I]
                yield hp + f"mlp.experts.{e}.up_proj.weight", gu[e, I:]
                yield hp + f"mlp.experts.{e}.down_proj.weight", dn[e]
        elif apertus:
            yield hp + "mlp.up_proj.weight", params[p + "mlp.up_proj"]
            yield hp + "mlp.down_proj.weight", params[p + "mlp.down_proj"]
            yield hp + "mlp.act_fn.alpha_p", params[p + "mlp.act_alpha_p"]
            yield hp + "mlp.act_fn.alpha_n", params[p + "mlp.act_alpha_n"]
        else:
            gu = params[p + "mlp.gate_up_proj"]
            I = cfg.intermediate_size
            yield hp + "mlp.gate_proj.weight", gu[:I]
            yield hp + "mlp.up_proj.weight", gu[I:]
            yield hp + "mlp.down_proj.weight", params[p + "mlp.down_proj"]
    if "norm" in params:
        yield "model.norm.weight", params["norm"]
    if "score" in params:
        yield "score.weight", params["score"]
    if "lm_head" in params and params.get("lm_head") is not None:
        yield "lm_head.weight", params["lm_head"]


def hf_to_native_state_dict(cfg: ModelConfig, sd: dict) -> dict:
    """Fuse q/k/v and gate/up tensors of an HF state dict into this model's parameter names."""
    out = {}
    g = sd.get
    if "model.embed_tokens.weight" in sd:
        out["embed_tokens"] = sd["model.embed_tokens.weight"]
    for i in range(cfg.num_hidden_layers):
        hp, p = f"model.layers.{i}.", f"layers.{i}."
        apertus = getattr(cfg, "mlp_act", "swiglu") == "xielu"
        n1, n2 = ("attention_layernorm.weight", "feedforward_layernorm.weight") if apertus else ("input_layernorm.weight", "post_attention_layernorm.weight")
        if hp + n1 not in sd:
            continue
        out[p + "input_layernorm"] = sd[hp + n1]
        out[p + "post_attention_layernorm"] = sd[hp + n2]
        out[p + "self_attn.qkv_proj"] = torch.cat([sd[hp + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)
        if cfg.attention_bias and hp + "self_attn.q_proj.bias" in sd:
            out[p + "self_attn.qkv_bias"] = torch.cat([sd[hp + f"self_attn.{n}_proj.bias"] for n in "qkv"], 0)
        out[p + "self_attn.o_proj"] = sd[hp + "self_attn.o_proj.weight"]
        if cfg.qk_norm:
            out[p + "self_attn.q_norm"] = sd[hp + "self_attn.q_norm.weight"]
            out[p + "self_attn.k_norm"] = sd[hp + "self_attn.k_norm.weight"]
        if cfg.is_moe:
            out[p + "mlp.router"] = sd[hp + "mlp.gate.weight"]
            out[p + "mlp.experts_gate_up"] = torch.stack(
                [torch.cat([sd[hp + f"mlp.experts.{e}.gate_proj.weight"], sd[hp + f"mlp.experts.{e}.up_proj.weight"]], 0)
                 for e in range(cfg.num_experts)], 0)
            out[p + "mlp.experts_down"] = torch.stack([sd[hp + f"mlp.experts.{e}.down_proj.weight"] for e in range(cfg.num_experts)], 0)
        elif apertus:
            out[p + "mlp.up_proj"] = sd[hp + "mlp.up_proj.weight"]
            out[p + "mlp.down_proj"] = sd[hp + "mlp.down_proj.weight"]
            out[p + "mlp.act_alpha_p"] = sd[hp + "mlp.act_fn.alpha_p"].reshape(1)
            out[p + "mlp.act_alpha_n"] = sd[hp + "mlp.act_fn.alpha_n"].reshape(1)
        else:
            out[p + "mlp.gate_up_proj"] = torch.cat([sd[hp + "mlp.gate_proj.weight"], sd[hp + "mlp.up_proj.weight"]], 0)
            out[p + "mlp.down_proj"] = sd[hp + "mlp.down_proj.weight"]
    if "model.norm.weight" in sd:
        out["norm"] = sd["model.norm.weight"]
    if g("lm_head.weight") is not None and not cfg.tie_word_embeddings and not cfg.value_head:
        out["lm_head"] = sd["lm_head.weight"]
    if g("score.weight") is not None:
        out["score"] = sd["score.weight"]
    return out
