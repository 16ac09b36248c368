"""3-D parallel training engine: tensor parallel × pipeline parallel × data parallel (sharded optimizer over DP).

Same ``BaseEngine`` contract as the sharded-DP engine, selected with ``strategy: megatron``. The reference delegates
this to Megatron-Core (``verl/workers/engine/megatron/transformer_impl.py:260-340`` process groups and model build,
``:885-971`` pipeline schedule, ``:981-1009`` weight export); here it is self-contained:

* rank layout ``rank = pp_rank · (dp·cp·tp) + dp_rank · (cp·tp) + cp_rank · tp + tp_rank`` (TP fastest so a TP group sits on
  adjacent GPUs, the context-parallel ranks of a replica next);
* TP: column/row-parallel projections with the f/g autograd pair, vocabulary-parallel embedding and a
  vocabulary-parallel fused lm_head→log-prob kernel (one [3, T] all-gather instead of materialised logits);
* PP: contiguous layer ranges, 1F1B schedule over the micro-batches with paired isend/irecv, activations ``[T, H]``;
* CP: the ranks of a context-parallel group hold the same micro-batch and each a slice of its packed token stream; attention
  all-gathers K/V (``verl_b200.parallel.context_parallel``), the last stage gathers the per-token outputs. For parameters CP
  ranks behave like data-parallel ranks: gradients are averaged and the optimizer state is sharded over the DP×CP group;
* DP: gradients are averaged and the fp32 master/Adam state is sharded over the DP group (distributed optimizer),
  reusing the flat-buffer machinery of the sharded-DP engine; the gradient norm is combined over TP×PP with
  replicated parameters counted once;
* weight export gathers TP shards and broadcasts across stages so every rank can yield full HF-named tensors.
"""

from __future__ import annotations

import os
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from verl_b200 import ops
from verl_b200.models.parallel_model import (local_model_config, local_to_global_name, shard_param, stage_layer_range, tp_rule,
                                             unshard_param)
from verl_b200.models.transformer import DecoderLM, native_to_hf_tensors
from verl_b200.ops.lm_head import vocab_parallel_logprob
from verl_b200.parallel.tp import copy_to_tp

from verl_b200.utils.metric import AggregationType, Metric
from verl_b200.utils.seqlen_balancing import restore_dynamic_batch
from verl_b200.workers.engine.base import EngineRegistry
from verl_b200.workers.engine.fsdp.engine import _DTYPES, FlatParamStore, FSDPEngine, _to_device, cfg_get
from verl_b200.workers.utils.padding import response_gather_index

__all__ = ["MegatronEngine", "MegatronEngineWithValueHead"]


def _new_groups(rank: int, rank_lists: list[list[int]]):
    """Create every group of a family (all ranks must call new_group for all of them) and return (mine, my ranks)."""
    mine, mine_ranks = None, None
    for ranks in rank_lists:
        g = dist.new_group(ranks)
        if rank in ranks:
            mine, mine_ranks = g, ranks
    return mine, mine_ranks


class _VirtualChunks(torch.nn.Module):
    """The model chunks one pipeline rank holds under virtual pipeline parallelism (chunk c = virtual stage c * pp + pp_rank)."""

    def __init__(self, chunks):
        super().__init__()
        self.chunks = torch.nn.ModuleList(chunks)

    @property
    def layers(self):
        return [layer for ch in self.chunks for layer in ch.layers]

    @property
    def embed_tokens(self):
        return next(ch.embed_tokens for ch in self.chunks if getattr(ch, "embed_tokens", None) is not None)

    def set_tp_group(self, *args, **kwargs):
        for ch in self.chunks:
            ch.set_tp_group(*args, **kwargs)

    def __setattr__(self, name, value):
        if name in ("gradient_checkpointing", "sp_group"):        # per-chunk switches set on the whole model by the engine
            for ch in self.chunks:
                setattr(ch, name, value)
            return
        super().__setattr__(name, value)


@EngineRegistry.register(model_type="language_model", backend=["megatron"], device=["cuda", "cpu"])
class MegatronEngine(FSDPEngine):
    def __init__(self, model_config, engine_config=None, optimizer_config=None, checkpoint_config=None):
        super().__init__(model_config, engine_config, optimizer_config, checkpoint_config)
        ec = self.engine_config
        self.tp_size = int(cfg_get(ec, "tensor_model_parallel_size", 1) or 1)
        # Megatron sequence parallelism: token-sharded stream between the TP regions, all-gather / reduce-scatter fused
        # into the projections. Off unless asked for (the reference's megatron.yaml turns it on by default).
        self.tp_sp = bool(cfg_get(ec, "sequence_parallel", False)) and self.tp_size > 1
        self.pp_size = int(cfg_get(ec, "pipeline_model_parallel_size", 1) or 1)
        for key in ("expert_model_parallel_size",):
            v = cfg_get(ec, key, None)
            if v not in (None, 1, 0):
                raise NotImplementedError(f"{key}={v} is not supported by this engine yet")
        # virtual pipeline stages: every pipeline rank holds `vpp` model chunks (virtual stage s = chunk * pp + pp_rank owns the
        # s-th of pp * vpp contiguous layer blocks) and runs the interleaved 1F1B schedule, which shrinks the pipeline bubble by vpp
        self.vpp = int(cfg_get(ec, "virtual_pipeline_model_parallel_size", None) or 1)
        if self.vpp > 1 and self.pp_size < 2:
            raise ValueError("virtual_pipeline_model_parallel_size > 1 needs pipeline_model_parallel_size > 1")
        self.cp_size = int(cfg_get(ec, "context_parallel_size", 1) or 1)
        self._cp_zigzag = self.cp_size > 1 and bool(cfg_get(ec, "context_parallel_zigzag", False))
        self._dynamic_cp = False
        mp = self.tp_size * self.pp_size * self.cp_size
        assert self.world % mp == 0, "world size must be a multiple of tp·pp·cp"
        self.sp_size = 1
        self.dp_size = self.world // mp
        tp, cp, dp = self.tp_size, self.cp_size, self.dp_size
        self.tp_rank = self.rank % tp
        self.cp_rank = (self.rank // tp) % cp
        self.dp_rank = (self.rank // (tp * cp)) % dp
        self.pp_rank = self.rank // (tp * cp * dp)
        # parameters are replicated over DP×CP: that is the group the gradients are averaged over and the optimizer state is cut over
        self.fsdp_size, self.fsdp_rank, self.ddp_size = dp * cp, self.dp_rank * cp + self.cp_rank, 1

    # ------------------------------------------------------------------ groups
    def _build_groups(self):
        tp, cp, dp, pp, W = self.tp_size, self.cp_size, self.dp_size, self.pp_size, self.world
        self.tp_group = self.pp_group = self.mp_group = self.dp_group = self.embed_group = self.cp_group = None
        self.fsdp_group = self.ddp_group = self.sp_group = None
        self.sp_rank = 0
        stage = dp * cp * tp                                  # ranks per pipeline stage
        rk = lambda p, d, c, t: p * stage + d * cp * tp + c * tp + t      # noqa: E731
        self.prev_rank = self.rank - stage if self.pp_rank > 0 else None
        self.next_rank = self.rank + stage if self.pp_rank < pp - 1 else None
        self.mp_ranks = [rk(p, self.dp_rank, self.cp_rank, t) for p in range(pp) for t in range(tp)]
        self.pp_ranks = [rk(p, self.dp_rank, self.cp_rank, self.tp_rank) for p in range(pp)]
        if W == 1:
            return
        if tp > 1:
            self.tp_group, _ = _new_groups(self.rank, [list(range(b, b + tp)) for b in range(0, W, tp)])
        if cp > 1:
            self.cp_group, _ = _new_groups(self.rank, [[rk(p, d, c, t) for c in range(cp)] for p in range(pp) for d in range(dp) for t in range(tp)])
        if dp > 1:
            self.dp_group, _ = _new_groups(self.rank, [[rk(p, d, c, t) for d in range(dp)] for p in range(pp) for c in range(cp) for t in range(tp)])
        if pp > 1:
            self.pp_group, _ = _new_groups(self.rank, [[rk(p, d, c, t) for p in range(pp)] for d in range(dp) for c in range(cp) for t in range(tp)])
        if tp * pp > 1:
            self.mp_group, _ = _new_groups(self.rank, [[rk(p, d, c, t) for p in range(pp) for t in range(tp)] for d in range(dp) for c in range(cp)])
        if pp > 1 and self.vpp > 1:
            # interleaved schedule: four kinds of messages travel between neighbouring ranks (activations to the next rank, activations
            # wrapping from the last rank to the first, and the two gradient directions). Each kind gets a communicator of its own so
            # that a send of one kind never queues behind a receive of another on the same stream.
            lists = [[rk(p, d, c, t) for p in range(pp)] for d in range(dp) for c in range(cp) for t in range(tp)]
            self._p2p_groups = {kind: _new_groups(self.rank, lists)[0] for kind in ("f", "fw", "b", "bw")}
        if pp > 1:   # first and last stage of each pipeline: gradient sum of tied input/output embeddings
            self.embed_group, _ = _new_groups(self.rank, [[rk(0, d, c, t), rk(pp - 1, d, c, t)] for d in range(dp) for c in range(cp) for t in range(tp)])
        if cp == 1:
            self.fsdp_group = self.dp_group
        elif dp * cp > 1:
            self.fsdp_group, _ = _new_groups(self.rank, [[rk(p, d, c, t) for d in range(dp) for c in range(cp)] for p in range(pp) for t in range(tp)])

    # ------------------------------------------------------------------ build
    def initialize(self):
        cfg = self._resolve_model_config()
        self.cfg = cfg
        if cfg.vision:
            raise NotImplementedError("vision-language models run in the sharded data-parallel engine (strategy=fsdp), not under tensor/pipeline parallelism")
        if not hasattr(self.model_config, "num_hidden_layers") and int(cfg_get(self.model_config, "lora_rank", 0) or 0) > 0:
            raise NotImplementedError("low-rank adapters are trained by the sharded data-parallel engine (strategy=fsdp); the tensor/pipeline-parallel "
                                      "engine would silently train every weight, so model.lora_rank > 0 is refused here")
        dt_name = cfg_get(self.engine_config, "model_dtype", None) or (cfg.torch_dtype if self.device.type == "cpu" else "bfloat16")
        self.dtype = _DTYPES.get(str(dt_name), torch.bfloat16)
        seed = int(cfg_get(self.engine_config, "seed", 0))
        self._build_groups()
        tp, pp = self.tp_size, self.pp_size
        self.layer_range = stage_layer_range(cfg.num_hidden_layers, pp, self.pp_rank)
        self.is_first, self.is_last = self.pp_rank == 0, self.pp_rank == pp - 1
        self.local_cfg = local_model_config(cfg, tp)
        # the full model is materialised once (same seed everywhere, or the HF checkpoint) and cut into this rank's piece
        full = DecoderLM(cfg, dtype=self.dtype, device=self.device, init=True, seed=seed)
        path = cfg_get(self.model_config, "path", None) if not hasattr(self.model_config, "num_hidden_layers") else None
        if path and os.path.isdir(os.path.expanduser(path)):
            from verl_b200.models.hf_io import load_hf_weights

            load_hf_weights(full, os.path.expanduser(path), strict=not cfg.value_head)
        if tp * pp == 1:
            self.model = full
        else:
            if self.vpp > 1:
                nv = pp * self.vpp
                if cfg.num_hidden_layers < nv:
                    raise ValueError(f"{cfg.num_hidden_layers} layers cannot fill {pp} x {self.vpp} virtual pipeline stages")
                chunks = []
                for c in range(self.vpp):
                    vs = c * pp + self.pp_rank
                    chunks.append(DecoderLM(self.local_cfg, dtype=self.dtype, device=self.device, init=False,
                                            layer_range=stage_layer_range(cfg.num_hidden_layers, nv, vs), pre_process=vs == 0, post_process=vs == nv - 1))
                self.model = _VirtualChunks(chunks)
                self.layer_range = [ch.layer_offset for ch in chunks]
            else:
                self.model = DecoderLM(self.local_cfg, dtype=self.dtype, device=self.device, init=False, layer_range=self.layer_range,
                                       pre_process=self.is_first, post_process=self.is_last)
            full_params = dict(full.named_parameters())
            with torch.no_grad():
                for name, p in self.model.named_parameters():
                    g = self._gname(name)
                    p.copy_(shard_param(g, full_params[g], cfg, self.tp_rank, tp))
            del full, full_params
            if tp > 1:
                tp_ctx = None
                if self.tp_sp and self.device.type == "cuda":
                    from verl_b200.parallel.tp import TPContext, fused_comm_enabled

                    if fused_comm_enabled():
                        max_tok = int(cfg_get(self.engine_config, "sequence_parallel_max_tokens", 32768))
                        tp_ctx = TPContext(self.tp_group, self._tp_host_group(), max_tokens=max_tok, hidden=cfg.hidden_size, max_out=cfg.hidden_size)
                self.model.set_tp_group(self.tp_group, self.tp_rank * self.local_cfg.vocab_size, sequence_parallel=self.tp_sp, tp_ctx=tp_ctx)
        self.model.gradient_checkpointing = bool(cfg_get(self.model_config, "enable_gradient_checkpointing", False))
        if self.cp_size > 1:
            self.model.sp_group = self.cp_group
            for layer in self.model.layers:
                layer.self_attn.sp_mode = "context"
        self.store = FlatParamStore(self.model, self.fsdp_size, self.fsdp_rank)
        if self.fsdp_size > 1:
            dist.broadcast(self.store.flat, src=self.pp_rank * self.fsdp_size * tp + self.tp_rank, group=self.fsdp_group)
        self._symm_params = self._symm_grads = None
        self._dup_ranges = self._replicated_ranges()
        if not self.forward_only:
            self._build_optimizer()
        from verl_b200.utils.checkpoint.megatron_checkpoint_manager import MegatronCheckpointManager

        self.checkpoint_manager = MegatronCheckpointManager(self, self.checkpoint_config)
        if self._param_offload:
            self.to("cpu", model=True, optimizer=False, grad=False)
        if self._optimizer_offload and not self.forward_only:
            self.to("cpu", model=False, optimizer=True, grad=True)

    def _gname(self, name: str) -> str:
        """Parameter name of this rank's model piece → name in the full model."""
        if self.vpp > 1:
            _, c, rest = name.split(".", 2)
            return local_to_global_name(rest, self.model.chunks[int(c)].layer_offset)
        return local_to_global_name(name, self.model.layer_offset)

    def _chunk(self, chunk: Optional[int]):
        return self.model if self.vpp == 1 else self.model.chunks[chunk or 0]

    def _virtual_stage(self, chunk: Optional[int]) -> int:
        return (chunk or 0) * self.pp_size + self.pp_rank

    def _tp_host_group(self):
        """gloo twin of this rank's TP group (pointer tables of the symmetric buffers travel through host memory)."""
        if getattr(self, "_tp_host", None) is None:
            tp = self.tp_size
            self._tp_host, _ = None, None
            for b in range(0, self.world, tp):
                g = dist.new_group(list(range(b, b + tp)), backend="gloo")
                if b <= self.rank < b + tp:
                    self._tp_host = g
        return self._tp_host

    def _pack(self, mb: dict):
        pb, labels = super()._pack(mb)
        if not self.tp_sp:
            return pb, labels
        # the token axis is split over the TP ranks: round the packed length up with one dummy sequence
        from verl_b200.models.transformer import PackedBatch

        T = pb.input_ids.shape[0]
        pad = (-T) % self.tp_size
        if pad == 0:
            return pb, labels
        dev = pb.input_ids.device
        ids = torch.cat([pb.input_ids, torch.zeros(pad, dtype=pb.input_ids.dtype, device=dev)])
        pos = torch.cat([pb.position_ids, torch.arange(pad, dtype=pb.position_ids.dtype, device=dev)])
        cu_cpu = torch.cat([pb.cu_seqlens_cpu, torch.tensor([T + pad], dtype=pb.cu_seqlens_cpu.dtype)])
        lab = torch.cat([labels, torch.zeros(pad, dtype=labels.dtype, device=dev)])
        return PackedBatch(ids, pos, cu_cpu.to(dev), cu_cpu, max(pb.max_seqlen, pad), pb.routed_experts), lab

    def _replicated_ranges(self) -> list[tuple[int, int, float]]:
        """(start, stop, weight) ranges of the flat buffer whose squared gradient must be down-weighted in the global
        norm because the parameter exists on several model-parallel ranks (TP-replicated norms, tied embeddings)."""
        out = []
        tied_copy = self.pp_size > 1 and self.cfg.tie_word_embeddings and not self.cfg.value_head
        for name, p, off in zip(self.store.names, self.store.params, self.store.offsets):
            g = self._gname(name)
            copies = 1
            if self.tp_size > 1 and tp_rule(g, self.cfg) is None:
                copies *= self.tp_size
            if tied_copy and g == "embed_tokens":
                copies *= 2
            if copies > 1:
                out.append((off, off + p.numel(), 1.0 / copies))
        return out

    # ------------------------------------------------------------------ contract
    def is_mp_src_rank_with_outputs(self) -> bool:
        return self.tp_rank == 0 and self.cp_rank == 0 and self.pp_rank == self.pp_size - 1

    def _micro_batch_indices(self, seq_lens, meta):
        from verl_b200.utils.seqlen_balancing import rearrange_micro_batches

        n = seq_lens.numel()
        if meta.get("use_dynamic_bsz", False):
            return rearrange_micro_batches(seq_lens.cpu(), int(meta["max_token_len_per_gpu"]), dp_group=self.dp_group)
        mbs = int(meta.get("micro_batch_size_per_gpu", 0) or n)
        return [list(range(i, min(n, i + mbs))) for i in range(0, n, mbs)]

    # ------------------------------------------------------------------ one stage
    def _cp_slice(self, pb, labels):
        """This context-parallel rank's slice of the packed micro-batch (contiguous or zig-zag placement): the local
        ``PackedBatch`` keeps the cu_seqlens of the whole stream (attention needs them), ``rows`` are the global token indices
        of the local rows and ``t_pad`` the padded stream length."""
        from verl_b200.models.transformer import PackedBatch
        from verl_b200.parallel.context_parallel import zigzag_permutation

        cp, r = self.cp_size, self.cp_rank
        T = pb.input_ids.shape[0]
        unit = cp * (2 if self._cp_zigzag else 1) * (self.tp_size if self.tp_sp else 1)
        pad = (-T) % unit
        ids, pos, lab = pb.input_ids, pb.position_ids, labels
        if pad:
            ids, lab = torch.nn.functional.pad(ids, (0, pad)), torch.nn.functional.pad(lab, (0, pad))
            pos = torch.cat([pos, torch.arange(pad, device=pos.device, dtype=pos.dtype)])
        tl = (T + pad) // cp
        if self._cp_zigzag:
            rows = zigzag_permutation(T + pad, cp).to(ids.device)[r * tl:(r + 1) * tl]
        else:
            rows = torch.arange(r * tl, (r + 1) * tl, device=ids.device)
        pbl = PackedBatch(ids.index_select(0, rows), pos.index_select(0, rows), pb.cu_seqlens, pb.cu_seqlens_cpu, pb.max_seqlen, None)
        pbl.cp_zigzag = self._cp_zigzag
        return pbl, lab.index_select(0, rows), T + pad

    def _stage_forward(self, mb: dict, meta: dict, h_in: Optional[torch.Tensor], chunk: Optional[int] = None):
        """Runs this stage (model chunk ``chunk`` under virtual pipeline parallelism) on one micro-batch. Returns (stream or None,
        model_output dict on the last stage)."""
        if self.cp_size > 1:
            return self._stage_forward_cp(mb, meta, h_in, chunk)
        pb, labels = self._pack(mb)
        model = self._chunk(chunk)
        h = model.forward_hidden(pb, h_in)
        if not model.post_process:
            return h, None
        R = mb["responses"].shape[1]
        idx, valid = response_gather_index(mb["attention_mask"], R)
        out: dict[str, torch.Tensor] = {}
        if self.cfg.value_head:
            vals = torch.nn.functional.linear(h, model.score).squeeze(-1).float()
            out["values"] = torch.where(valid, vals[idx.reshape(-1)].reshape(idx.shape), torch.zeros((), device=vals.device))
            return None, out
        temperature = float(meta.get("temperature", 1.0))
        need_entropy = bool(meta.get("calculate_entropy", False))
        sel = idx[valid]
        h_sel, lab_sel = h.index_select(0, sel), labels.index_select(0, sel)
        if self.tp_size > 1:
            lp, ent = vocab_parallel_logprob(copy_to_tp(h_sel, self.tp_group), model.output_weight, lab_sel, temperature,
                                             need_entropy, self.tp_group, model.vocab_offset)
        else:
            lp, ent = ops.linear_logprob_entropy(h_sel, model.output_weight, lab_sel, temperature, need_entropy)
        full = torch.zeros(idx.shape, dtype=torch.float32, device=h.device)
        out["log_probs"] = full.masked_scatter(valid, lp.float())
        if ent is not None:
            out["entropy"] = torch.zeros_like(full).masked_scatter(valid, ent.float())
        if meta.get("score_centering") or meta.get("distillation") or meta.get("return_topk"):
            # top-k head passes (score centering, distillation) need the whole vocabulary on one rank
            if self.tp_size > 1:
                raise NotImplementedError("score centering / distillation heads are not available with a vocabulary-parallel lm_head; "
                                          "use tensor_model_parallel_size=1 for this role or the sharded-DP engine")
            self._score_centering_terms(out, mb, meta, h_sel, valid, temperature)
        return None, out

    def _stage_forward_cp(self, mb: dict, meta: dict, h_in: Optional[torch.Tensor], chunk: Optional[int] = None):
        """The same with context parallelism: the stage works on this rank's token slice; on the last stage the per-token
        outputs of the slices are gathered over the CP group (gradient scaled by cp: the DP×CP average then counts every
        token once) and put back into stream order before the response window is cut out."""
        from verl_b200.parallel.ulysses import gather_outputs_and_unpad

        pb, labels = FSDPEngine._pack(self, mb)
        T = pb.input_ids.shape[0]
        pbl, lab_l, t_pad = self._cp_slice(pb, labels)
        model = self._chunk(chunk)
        h = model.forward_hidden(pbl, h_in)
        if not model.post_process:
            return h, None
        R = mb["responses"].shape[1]
        idx, valid = response_gather_index(mb["attention_mask"], R)
        out: dict[str, torch.Tensor] = {}

        def to_stream(x_local):
            x = gather_outputs_and_unpad(x_local.float(), 0, None, 0, grad_scaler=True, group=self.cp_group)
            if self._cp_zigzag:
                from verl_b200.parallel.context_parallel import zigzag_permutation

                x = x.index_select(0, torch.argsort(zigzag_permutation(t_pad, self.cp_size).to(x.device)))
            return x[:T]

        zero = torch.zeros(idx.shape, dtype=torch.float32, device=h.device)
        if self.cfg.value_head:
            vals = to_stream(torch.nn.functional.linear(h, model.score).squeeze(-1))
            out["values"] = torch.where(valid, vals[idx.reshape(-1)].reshape(idx.shape), zero)
            return None, out
        temperature = float(meta.get("temperature", 1.0))
        need_entropy = bool(meta.get("calculate_entropy", False))
        if self.tp_size > 1:
            lp, ent = vocab_parallel_logprob(copy_to_tp(h, self.tp_group), model.output_weight, lab_l, temperature, need_entropy,
                                             self.tp_group, model.vocab_offset)
        else:
            lp, ent = ops.linear_logprob_entropy(h, model.output_weight, lab_l, temperature, need_entropy)
        out["log_probs"] = torch.where(valid, to_stream(lp)[idx.reshape(-1)].reshape(idx.shape), zero)
        if ent is not None:
            out["entropy"] = torch.where(valid, to_stream(ent)[idx.reshape(-1)].reshape(idx.shape), zero)
        if meta.get("score_centering") or meta.get("distillation") or meta.get("return_topk"):
            raise NotImplementedError("score centering / distillation heads are not available under context parallelism in this engine")
        return None, out

    # ------------------------------------------------------------------ p2p
    def _exchange(self, send: Optional[torch.Tensor], send_to: Optional[int], recv_shape, recv_from: Optional[int]):
        """One paired isend/irecv step with the neighbouring stages; returns the received tensor (or None)."""
        reqs, recv = [], None
        if send is not None and send_to is not None:
            reqs.append(dist.P2POp(dist.isend, send.contiguous(), send_to))
        if recv_from is not None and recv_shape is not None:
            recv = torch.empty(recv_shape, dtype=self.dtype, device=self.device)
            reqs.append(dist.P2POp(dist.irecv, recv, recv_from))
        if reqs:
            for r in dist.batch_isend_irecv(reqs):
                r.wait()
        return recv

    # ------------------------------------------------------------------ interleaved schedule (virtual pipeline stages)
    def _run_interleaved(self, m: int, train: bool, run_forward, run_backward, shape) -> None:
        """Interleaved 1F1B over ``pp * vpp`` virtual stages. Micro-batches go through in groups of ``pp``; step k of the forward
        order is (chunk, micro-batch) = ((k % (pp*vpp)) // pp, (k // (pp*vpp)) * pp + k % pp), the backward order is the same with
        the chunks reversed. A rank runs ``(pp - rank - 1) * 2 + (vpp - 1) * pp`` forwards ahead, then alternates one forward and one
        backward, then drains. When the number of micro-batches is not a multiple of ``pp`` the missing ones of the last group are
        skipped by every rank alike (a valid schedule with steps removed stays valid). Sends are asynchronous and every kind of
        message has its own communicator, receives are waited for where the data is needed; both ends of a link issue their sends
        and receives in the same order, so no tags are needed."""
        pp, v, r = self.pp_size, self.vpp, self.pp_rank
        nv = pp * v
        groups = -(-m // pp)
        total = groups * pp * v
        nxt, prv = self.pp_ranks[(r + 1) % pp], self.pp_ranks[(r - 1) % pp]
        g = self._p2p_groups
        pending: list = []          # (work, tensor) of sends in flight: the tensors must outlive them

        def step_of(k, backward):
            c = (k % nv) // pp
            return (v - 1 - c if backward else c), (k // nv) * pp + k % pp

        def send(t, dst, kind):
            t = t.contiguous()
            pending.append((dist.isend(t, dst, group=g[kind]), t))

        def recv(shp, src, kind):
            t = torch.empty(shp, dtype=self.dtype, device=self.device)
            dist.irecv(t, src, group=g[kind]).wait()
            return t

        stash: dict = {}

        def forward(k):
            c, i = step_of(k, False)
            if i >= m:
                return
            vs = c * pp + r
            h_in = None
            if vs > 0:
                h_in = recv(shape(i), prv, "fw" if r == 0 else "f")
            h_in, stream, loss = run_forward(i, h_in, c)
            if vs < nv - 1:
                send(stream.detach(), nxt, "fw" if r == pp - 1 else "f")
            if train:
                stash[(c, i)] = (h_in, stream, loss)

        def backward(k):
            c, i = step_of(k, True)
            if i >= m:
                return
            vs = c * pp + r
            h_in, stream, loss = stash.pop((c, i))
            out_grad = None
            if vs < nv - 1:
                out_grad = recv(shape(i), nxt, "bw" if r == pp - 1 else "b")
            in_grad = run_backward(h_in, stream, loss, out_grad)
            if vs > 0:
                send(in_grad, prv, "bw" if r == 0 else "b")

        if not train:
            for k in range(total):
                forward(k)
        else:
            warm = min((pp - r - 1) * 2 + (v - 1) * pp, total)
            for k in range(warm):
                forward(k)
            for j in range(total - warm):
                forward(warm + j)
                backward(j)
            for j in range(total - warm, total):
                backward(j)
            assert not stash
        for w, _ in pending:
            w.wait()

    # ------------------------------------------------------------------ forward / backward over the pipeline
    def forward_backward_batch(self, data, loss_function: Optional[Callable], forward_only: bool = False) -> dict:
        batch = data.batch
        meta = dict(getattr(data, "meta_info", {}) or {})
        dev = self.device
        tensors = {k: (_to_device(v, dev) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        n = tensors["input_ids"].shape[0]
        seq_lens = tensors["attention_mask"].sum(-1)
        mb_indices = self._micro_batch_indices(seq_lens, meta)
        info: dict[str, Any] = {"dp_size": self.dp_size}
        train = not forward_only and loss_function is not None
        if train:
            ntok = tensors["response_mask"].sum().to(torch.float32) if "response_mask" in tensors else seq_lens.sum().to(torch.float32)
            cnt = torch.stack([ntok, torch.tensor(float(n), device=dev)])
            if self.dp_size > 1:
                dist.all_reduce(cnt, group=self.dp_group)
            info["batch_num_tokens"], info["global_batch_size"] = cnt[0], cnt[1]
            self._alloc_grads()
        self.model.train(not forward_only)

        def micro(i):
            it = torch.as_tensor(mb_indices[i], device=dev)
            return {k: (v.index_select(0, it) if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == n else v)
                    for k, v in tensors.items()}

        H = self.cfg.hidden_size
        ntoks = [int(seq_lens[torch.as_tensor(ix, device=seq_lens.device)].sum()) for ix in mb_indices]
        if self.cp_size > 1:   # stage boundaries carry this rank's slice of the padded stream (and 1/tp of it under sequence parallelism)
            unit = self.cp_size * (2 if self._cp_zigzag else 1) * (self.tp_size if self.tp_sp else 1)
            ntoks = [-(-t // unit) * unit // self.cp_size for t in ntoks]
            if self.tp_sp:
                ntoks = [t // self.tp_size for t in ntoks]
        elif self.tp_sp:      # stage boundaries carry this rank's 1/tp of the (padded) tokens
            ntoks = [-(-t // self.tp_size) for t in ntoks]
        m = len(mb_indices)
        outputs: dict[str, list[torch.Tensor]] = {}
        metrics: dict[str, Metric] = {}
        losses: list[float] = []

        def run_forward(i, h_in, chunk=None):
            mb = micro(i)
            if h_in is not None and train:
                h_in.requires_grad_(True)
            with (torch.enable_grad() if train else torch.no_grad()):
                stream, mo = self._stage_forward(mb, meta, h_in, chunk)
                loss = None
                if mo is not None:
                    if loss_function is not None:
                        mb_data = dict(mb)
                        mb_data.update(info)
                        loss, mt = loss_function(model_output=mo, data=mb_data, dp_group=self.dp_group)
                        losses.append(float(loss.detach()))
                        for k, v in mt.items():
                            if k in metrics:
                                metrics[k].append(v)
                            else:
                                metrics[k] = v if isinstance(v, Metric) else Metric(AggregationType.MEAN, v)
                    for k, v in mo.items():
                        outputs.setdefault(k, []).append(v.detach())
            return h_in, stream, loss

        def run_backward(h_in, stream, loss, out_grad):
            if loss is not None:
                loss.backward()
            else:
                torch.autograd.backward(stream, out_grad)
            return h_in.grad if h_in is not None else None

        first, last = self.is_first, self.is_last
        shape = lambda i: None if i is None or i >= m else (ntoks[i], H)
        if self.vpp > 1:
            self._run_interleaved(m, train, run_forward, run_backward, shape)
            if train:
                self.store.fold_autograd_grads()
                self._sync_replicated_grads()
        elif not train:
            for i in range(m):
                h_in = self._exchange(None, None, None if first else shape(i), self.prev_rank)
                _, stream, _ = run_forward(i, h_in)
                self._exchange(stream, self.next_rank, None, None)
        else:
            # 1F1B: `warm` forwards, then alternate one forward / one backward, then drain the backwards
            warm = min(self.pp_size - self.pp_rank - 1, m)
            steady = m - warm
            stash: list[tuple] = []
            fwd_i = 0
            for _ in range(warm):
                h_in = self._exchange(None, None, None if first else shape(fwd_i), self.prev_rank)
                stash.append((fwd_i,) + run_forward(fwd_i, h_in))
                self._exchange(stash[-1][2], self.next_rank, None, None)
                fwd_i += 1
            h_in = self._exchange(None, None, None if first or steady == 0 else shape(fwd_i), self.prev_rank) if steady > 0 else None
            for k in range(steady):
                stash.append((fwd_i,) + run_forward(fwd_i, h_in))
                cur = stash[-1]
                # send this forward's activations on, receive the gradient of the OLDEST pending micro-batch
                bi, b_in, b_stream, b_loss = stash.pop(0)
                out_grad = self._exchange(cur[2], self.next_rank, None if last else shape(bi), self.next_rank)
                in_grad = run_backward(b_in, b_stream, b_loss, out_grad)
                fwd_i += 1
                nxt = fwd_i if k < steady - 1 else None
                h_in = self._exchange(in_grad, self.prev_rank, None if first else shape(nxt), self.prev_rank)
            while stash:
                bi, b_in, b_stream, b_loss = stash.pop(0)
                out_grad = self._exchange(None, None, None if last else shape(bi), self.next_rank)
                in_grad = run_backward(b_in, b_stream, b_loss, out_grad)
                self._exchange(in_grad, self.prev_rank, None, None)
            self.store.fold_autograd_grads()
            self._sync_replicated_grads()
        model_output = {k: restore_dynamic_batch(torch.cat(v, 0), mb_indices) for k, v in outputs.items()}
        result = {"model_output": model_output, "loss": losses, "metrics": metrics}
        if self.pp_size > 1:
            result = self._broadcast_from_last_stage(result)
        return result

    def _broadcast_from_last_stage(self, result: dict) -> dict:
        """Outputs exist on the last stage only; the role workers expect them on every rank of the model-parallel group."""
        box = [result if self.is_last else None]
        if self.is_last:
            box[0] = {"model_output": {k: v.cpu() for k, v in result["model_output"].items()}, "loss": result["loss"], "metrics": result["metrics"]}
        dist.broadcast_object_list(box, src=self.pp_ranks[-1], group=self.pp_group)
        if self.is_last:
            return result
        got = box[0]
        got["model_output"] = {k: v.to(self.device) for k, v in got["model_output"].items()}
        return got

    def _sync_replicated_grads(self):
        """Gradients that are partial sums on each model-parallel rank although the parameter is replicated: the MoE router
        under expert tensor parallelism (its combine weights multiply partial expert outputs) and tied embeddings
        living on both the first and the last pipeline stage."""
        if self.tp_size > 1 and self.cfg.is_moe:
            for layer in self.model.layers:
                dist.all_reduce(layer.mlp.router.main_grad, group=self.tp_group)
        if self.tp_sp:
            # norms see a different token slice on every TP rank: their gradients are partial sums
            for name, p in self.model.named_parameters():
                if tp_rule(self._gname(name), self.cfg) is None and getattr(p, "main_grad", None) is not None \
                        and not name.endswith("router"):
                    dist.all_reduce(p.main_grad, group=self.tp_group)
        if self.pp_size > 1 and self.cfg.tie_word_embeddings and not self.cfg.value_head and (self.is_first or self.is_last):
            dist.all_reduce(self.model.embed_tokens.main_grad, group=self.embed_group)

    # ------------------------------------------------------------------ optimizer hooks
    def _sumsq_across_model_parallel(self, sumsq: torch.Tensor, gshard: torch.Tensor) -> torch.Tensor:
        if self.tp_size * self.pp_size == 1:
            return sumsq
        s = self.store
        lo = self.fsdp_rank * s.shard_size if gshard.numel() == s.shard_size and self.fsdp_size > 1 else 0
        corr = torch.zeros(1, dtype=torch.float32, device=gshard.device)
        for a, b, w in self._dup_ranges:
            a2, b2 = max(a, lo), min(b, lo + gshard.numel())
            if b2 > a2:
                corr += (1.0 - w) * gshard[a2 - lo : b2 - lo].float().pow(2).sum()
        if self.fsdp_size > 1:
            dist.all_reduce(corr, group=self.fsdp_group)
        total = (sumsq.reshape(1).float() - corr).clone()
        dist.all_reduce(total, group=self.mp_group)
        if sumsq.data_ptr() != total.data_ptr():
            sumsq.copy_(total.reshape(sumsq.shape))
        return sumsq

    # ------------------------------------------------------------------ weights out
    def get_per_tensor_param(self, **kwargs):
        """(HF name, full tensor) pairs on every rank: TP shards are all-gathered inside the owning stage and the result
        is broadcast along the pipeline (the reference's Megatron-Bridge export does the same TP gather + PP broadcast:
        verl/workers/engine/megatron/transformer_impl.py:981-1009)."""
        if not self.store.flat.is_cuda and self.device.type == "cuda":
            self.to("cuda", model=True, optimizer=False, grad=False)
        if self.tp_size * self.pp_size == 1:
            return self.model.hf_named_tensors(), None
        return self._gathered_hf_tensors(), None

    def _gathered_hf_tensors(self):
        cfg, tp, pp = self.cfg, self.tp_size, self.pp_size
        local = {self._gname(n): p for n, p in self.model.named_parameters()}
        # every rank walks the same global list; the tied copy of the embedding on the last stage is skipped
        probe = DecoderLM(cfg, dtype=self.dtype, device="meta", init=False)
        full_shapes = {n: tuple(p.shape) for n, p in probe.named_parameters()}
        owner_stage = {}
        for n in full_shapes:
            if n.startswith("layers."):
                li = int(n.split(".")[1])
                nv = pp * self.vpp          # virtual stage s lives on pipeline rank s % pp
                owner_stage[n] = next(s for s in range(nv) if li in stage_layer_range(cfg.num_hidden_layers, nv, s)) % pp
            else:
                owner_stage[n] = 0 if n == "embed_tokens" else pp - 1

        def full_tensor(n):
            st = owner_stage[n]
            t = None
            if st == self.pp_rank:
                mine = local[n].detach()
                if tp > 1 and tp_rule(n, cfg) is not None:
                    parts = [torch.empty_like(mine) for _ in range(tp)]
                    dist.all_gather(parts, mine.contiguous(), group=self.tp_group)
                    t = unshard_param(n, parts, cfg)
                else:
                    t = mine
            if pp > 1:
                if t is None:
                    t = torch.empty(full_shapes[n], dtype=self.dtype, device=self.device)
                t = t.contiguous()
                dist.broadcast(t, src=self.pp_ranks[st], group=self.pp_group)
            return t

        class _Lazy(dict):
            """Materialises a full tensor only when the name-mapping generator asks for it."""

            def __init__(self, names):
                super().__init__({n: None for n in names})

            def __getitem__(self, n):
                return full_tensor(n)

            def get(self, n, default=None):
                return full_tensor(n) if n in self else default

        return native_to_hf_tensors(cfg, _Lazy(full_shapes.keys()))


@EngineRegistry.register(model_type="value_model", backend=["megatron"], device=["cuda", "cpu"])
class MegatronEngineWithValueHead(MegatronEngine):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._value_head = True
