"""ZeRO-3 mode of the sharded data-parallel engine: the decoder's projection weights live row-sharded across the ranks and are
gathered on demand; the all-gather of the forward pass is fused into the consuming GEMM.

* Every rank keeps rows ``[r·N/W, (r+1)·N/W)`` of each ``[N, K]`` projection weight (qkv / o / gate_up / down) in a symmetric
  buffer that its peers can read; norms, biases, the embedding and the lm_head stay replicated.
* Forward ``y = x · gather(W)ᵀ``: one GEMM kernel whose B operand rows come from the owning ranks' memory over NVLink
  (``vb_gemm_allgather`` — the remote rows are copied into a local staging buffer once per call by dedicated copy warps while
  the tensor cores already work on the local rows). Without the kernels (CPU, ragged shard sizes) the weight is all-gathered.
* Backward: the weight is gathered again (NCCL), ``dx = dy · W`` and the full ``dW = dyᵀ · x`` are computed locally, ``dW`` is
  reduce-scattered and accumulated into the fp32 gradient of the local shard.
* Optimizer: AdamW runs on the local tensors only — no collective besides the gradient-norm sum and the all-reduce of the
  replicated tensors' gradients.

Reference: FSDP ``FULL_SHARD`` / ``fully_shard`` per decoder layer (``verl/workers/engine/fsdp/transformer_impl.py:389-498``,
``verl/utils/fsdp_utils.py:549-614``): all-gather of the flat parameters before forward and again before backward,
reduce-scatter of the gradients.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from verl_b200.ops import _ext
from verl_b200.ops.functional import gemm

__all__ = ["Zero3Shard", "zero3_linear", "SHARDED_LEAVES"]

SHARDED_LEAVES = ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")


class Zero3Shard:
    """Where a row-sharded weight lives: the symmetric buffer holding every rank's ``[rows, K]`` slice at ``byte_offset``."""

    __slots__ = ("group", "world", "rank", "rows", "in_features", "symm", "byte_offset", "ctx")

    def __init__(self, group, rows: int, in_features: int, symm=None, byte_offset: int = 0, ctx=None):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.in_features = rows, in_features
        self.symm, self.byte_offset, self.ctx = symm, byte_offset, ctx


class _GatherCtx:
    """Staging memory shared by all fused weight gathers of one engine (the largest full weight fits; calls are ordered by
    the stream). The kernel's chunk flags are counters that every call advances for the REMOTE 128-row chunks only, so a flag
    array and its epoch belong to one gathered height ``N`` (which fixes the chunk → owner map), not to the engine."""

    def __init__(self, max_elems: int, device):
        self.stage = torch.empty(max_elems, dtype=torch.bfloat16, device=device)
        self.device = device
        self._by_rows: dict[int, list] = {}
        self.calls = 0

    def next(self, rows_total: int):
        ent = self._by_rows.get(rows_total)
        if ent is None:
            ent = self._by_rows[rows_total] = [torch.zeros(rows_total // 128 + 8, dtype=torch.int32, device=self.device), 0]
        ent[1] += 1
        self.calls += 1
        return ent[0], ent[1]


def _gather_dim0(t: torch.Tensor, group) -> torch.Tensor:
    """All-gather along the first dimension (expert-parallel tensors ``[E/W, ...]`` → ``[E, ...]``)."""
    W = dist.get_world_size(group)
    full = torch.empty(t.shape[0] * W, *t.shape[1:], dtype=t.dtype, device=t.device)
    if t.is_cuda:
        dist.all_gather_into_tensor(full, t.contiguous(), group=group)
    else:
        dist.all_gather(list(full.chunk(W, 0)), t.contiguous(), group=group)
    return full


def _gather_rows(w_shard: torch.Tensor, sh: Zero3Shard) -> torch.Tensor:
    full = torch.empty(sh.rows * sh.world, sh.in_features, dtype=w_shard.dtype, device=w_shard.device)
    if w_shard.is_cuda:
        dist.all_gather_into_tensor(full, w_shard.contiguous(), group=sh.group)
    else:
        dist.all_gather(list(full.chunk(sh.world, 0)), w_shard.contiguous(), group=sh.group)
    return full


def _fused_ok(x: torch.Tensor, sh: Zero3Shard) -> bool:
    return (sh.symm is not None and x.is_cuda and x.dtype == torch.bfloat16 and _ext.available() and sh.rows % 128 == 0
            and sh.in_features % 64 == 0 and os.environ.get("VERL_B200_COMM", "native") == "native")


class _Zero3Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, bias, sh: Zero3Shard):
        ctx.sh = sh
        ctx.save_for_backward(x, w_shard)
        ctx.bias_ref = bias
        if _fused_ok(x, sh):
            from verl_b200.parallel.tp import TPContext

            flags, epoch = sh.ctx.next(sh.rows * sh.world)
            y = TPContext.weight_gather_linear(x.contiguous(), sh.symm, sh.rows, sh.in_features, sh.byte_offset, sh.ctx.stage, flags, epoch)
            return y if bias is None else y + bias
        return gemm(x, _gather_rows(w_shard, sh), bias=bias)

    @staticmethod
    def backward(ctx, dy):
        x, w_shard = ctx.saved_tensors
        sh: Zero3Shard = ctx.sh
        dy = dy.contiguous()
        w_full = _gather_rows(w_shard, sh)
        dx = gemm(dy, w_full, b_mn=True) if ctx.needs_input_grad[0] else None
        del w_full
        if ctx.needs_input_grad[1]:
            dw_full = gemm(dy, x, a_mn=True, b_mn=True, out=torch.zeros(sh.rows * sh.world, sh.in_features, dtype=torch.float32, device=dy.device),
                           accumulate=True)
            if dw_full.is_cuda:
                mine = torch.empty(sh.rows, sh.in_features, dtype=torch.float32, device=dy.device)
                dist.reduce_scatter_tensor(mine, dw_full, group=sh.group)
            else:
                dist.all_reduce(dw_full, group=sh.group)          # gloo has no reduce-scatter
                mine = dw_full[sh.rank * sh.rows:(sh.rank + 1) * sh.rows]
            w_shard.main_grad.add_(mine)
        db = None
        b = ctx.bias_ref
        if b is not None and ctx.needs_input_grad[2]:
            bsum = dy.float().sum(0)
            if getattr(b, "main_grad", None) is not None:
                b.main_grad.add_(bsum)
            else:
                db = bsum.to(b.dtype)
        return dx, None, db, None


def zero3_linear(x: torch.Tensor, w_shard: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ gather(w_shard)ᵀ (+ bias)`` for a weight tagged with a :class:`Zero3Shard` (``w_shard._zero3``)."""
    sh = w_shard._zero3
    if not torch.is_grad_enabled() or not (x.requires_grad or w_shard.requires_grad):
        if _fused_ok(x, sh):
            from verl_b200.parallel.tp import TPContext

            flags, epoch = sh.ctx.next(sh.rows * sh.world)
            y = TPContext.weight_gather_linear(x.contiguous(), sh.symm, sh.rows, sh.in_features, sh.byte_offset, sh.ctx.stage, flags, epoch)
            return y if bias is None else y + bias
        return gemm(x, _gather_rows(w_shard, sh), bias=bias)
    return _Zero3Linear.apply(x, w_shard, bias, sh)


# --------------------------------------------------------------------------------------------------------------------- engine
from verl_b200.workers.engine.base import EngineRegistry  # noqa: E402
from verl_b200.workers.engine.fsdp.engine import FlatParamStore, FSDPEngine, cfg_get  # noqa: E402

__all__ += ["Zero3Engine"]


def _is_sharded_name(name: str) -> bool:
    return name.startswith(("layers.", "language_model.layers.")) and name.rsplit(".", 1)[-1] in SHARDED_LEAVES


@EngineRegistry.register(model_type="language_model", backend=["fsdp_zero3"], device=["cuda", "cpu"])
class Zero3Engine(FSDPEngine):
    """Data-parallel engine with the decoder projections sharded by rows over ALL ranks (selected by ``zero3: true`` /
    ``reshard_after_forward: true`` in the engine config of the fsdp strategy), and/or the experts of a mixture-of-experts
    model spread over all ranks (``expert_parallel_size`` = world size): rank ``r`` owns experts ``[r·E/W, (r+1)·E/W)``, tokens
    travel to their experts by all-to-all (``verl_b200.ops.moe.moe_forward``). An expert's gradient is complete on its owner
    (the all-to-all backward brings every rank's contribution), so like the row shards it is only scaled by ``1/W``. Memory per rank: ``(sharded/W + replicated) · (2 + 4 + 12)`` bytes for working copy,
    fp32 gradients and AdamW state, against ``total · (2 + 4) + total/W · 12`` of the replicated-working-copy engine."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        assert self.sp_size == 1, "zero3 mode does not combine with sequence/context parallelism"
        self._param_offload = False            # the (already sharded) parameters stay on the device: peers read them in place
        self.fsdp_size = 1                     # the flat store holds only local tensors; nothing in it is sliced further
        ep = int(cfg_get(self.engine_config, "expert_parallel_size", 1) or 1)
        assert ep in (1, self.world), "expert_parallel_size must be 1 or the world size"
        self._ep = ep > 1
        self._shard_dense = bool(cfg_get(self.engine_config, "zero3", False) or cfg_get(self.engine_config, "reshard_after_forward", False))
        self._zero3_rows: dict[str, int] = {}

    def _build_groups(self):
        self.fsdp_group = self.ddp_group = self.sp_group = None
        self.fsdp_rank, self.ddp_size, self.sp_rank = 0, self.world, 0
        self.dp_size, self.dp_rank = self.world, self.rank
        self.dp_group = dist.group.WORLD if self.world > 1 else None
        self.shard_group = dist.group.WORLD if self.world > 1 else None

    # ---------------------------------------------------------------- placement
    def _place_parameters(self):
        assert not getattr(self.model, "lora_config", None), "zero3 mode does not support LoRA adapters"
        W, r = self.world, self.rank
        named = dict(self.model.named_parameters())
        if W > 1:
            for p in named.values():           # identical start everywhere (rank 0's values), before anything is sliced
                dist.broadcast(p.data, src=0)
        sharded = []
        if W > 1:
            for n, p in named.items():
                if self._ep and n.rsplit(".", 1)[-1] in ("experts_gate_up", "experts_down"):
                    assert p.shape[0] % W == 0, f"{p.shape[0]} experts do not divide over {W} ranks"
                    e_local = p.shape[0] // W
                    p._ep_full_shape = tuple(p.shape)
                    p.data = p.data[r * e_local:(r + 1) * e_local].clone()
                    self._zero3_rows[n] = e_local
                    continue
                if self._shard_dense and _is_sharded_name(n) and p.dim() == 2 and p.shape[0] % W == 0:
                    rows = p.shape[0] // W
                    full_shape = tuple(p.shape)
                    p.data = p.data[r * rows:(r + 1) * rows].clone()
                    p._zero3_full_shape = full_shape
                    self._zero3_rows[n] = rows
                    sharded.append(n)
        self.store = FlatParamStore(self.model, 1, 0, order_key=lambda np_: 0 if np_[0] in self._zero3_rows else 1)
        s = self.store
        self._n_shard_elems = min([o for n, o in zip(s.names, s.offsets) if n not in self._zero3_rows], default=s.total)
        self._symm_params = self._symm_grads = None
        symm = None
        use_symm = bool(cfg_get(self.engine_config, "use_symmetric_memory", True)) and os.environ.get("VERL_B200_COMM", "native") == "native"
        if use_symm and W > 1 and s.flat.is_cuda and s.flat.dtype == torch.bfloat16 and _ext.available():
            from verl_b200.parallel.symm_mem import SymmetricBuffer
            from verl_b200.single_controller.spmd import init_spmd_process_group

            host = init_spmd_process_group()
            symm = SymmetricBuffer(s.total * 2, host_group=host)
            new_flat = symm.tensor(torch.bfloat16, s.total)
            new_flat.copy_(s.flat)
            s.rebind(new_flat)
            self._zero3_symm = symm
            symm.barrier()
        gctx = None
        if symm is not None and sharded:
            full = [named[n]._zero3_full_shape for n in sharded]
            gctx = _GatherCtx(max(f[0] * f[1] for f in full), self.device)
        if self._ep:
            ep_ctx = None
            if (symm is not None and self.cfg.is_moe and self.world <= 8 and bool(cfg_get(self.engine_config, "fused_moe_dispatch", True))
                    and self.cfg.hidden_size % 128 == 0 and (2 * self.cfg.moe_intermediate_size) % 256 == 0):
                # dispatch and combine inside the grouped GEMMs: one token buffer + one slot buffer shared by all layers
                from verl_b200.ops.moe import FusedEPContext
                from verl_b200.single_controller.spmd import init_spmd_process_group

                max_tok = int(cfg_get(self.engine_config, "moe_max_tokens", 16384))
                ep_ctx = FusedEPContext(self.shard_group, init_spmd_process_group(), max_tok, self.cfg.hidden_size, self.cfg.num_experts_per_tok)
            self._ep_ctx = ep_ctx
            for layer in self.model.layers:
                if hasattr(layer.mlp, "ep_group"):
                    layer.mlp.ep_group = self.shard_group
                    layer.mlp.ep_ctx = ep_ctx
        for n, p, off in zip(s.names, s.params, s.offsets):
            if n in self._zero3_rows and p.dim() == 2:
                p._zero3 = Zero3Shard(self.shard_group, self._zero3_rows[n], p.shape[1], symm, off * 2, gctx)
        torch.cuda.empty_cache() if s.flat.is_cuda else None

    def to(self, device: str, model: bool = True, optimizer: bool = True, grad: bool = True):
        # sharded parameters are read by peers and must stay where they are; optimizer state and gradients may move
        return super().to(device, model=False, optimizer=optimizer, grad=grad)

    # ---------------------------------------------------------------- optimizer
    @torch.no_grad()
    def optimizer_step(self) -> float:
        s, W, ns = self.store, self.world, self._n_shard_elems
        assert s.grad is not None, "optimizer_step without gradients"
        g_sh, g_rep = s.grad[:ns], s.grad[ns:]
        if W > 1:
            # sharded tensors: the reduce-scatter in backward already summed over ranks → mean; replicated tensors: all-reduce
            g_sh.div_(W)
            if g_rep.is_cuda:
                dist.all_reduce(g_rep, op=dist.ReduceOp.AVG)
            else:
                dist.all_reduce(g_rep)
                g_rep.div_(W)
        native = s.grad.is_cuda and _ext.available()
        if native:
            self._sumsq.zero_()
            if ns:
                _ext.ops().sqnorm_(g_sh, self._sumsq)
            sumsq = self._sumsq
        else:
            sumsq = g_sh.float().pow(2).sum().reshape(1)
        if W > 1:
            dist.all_reduce(sumsq)
        if native:
            rep = torch.zeros_like(sumsq)
            _ext.ops().sqnorm_(g_rep, rep)
            sumsq.add_(rep)
        else:
            sumsq = sumsq + g_rep.float().pow(2).sum()
        grad_norm = self._adamw_update(s.grad, sumsq, native)
        if W > 1:
            # peers read this rank's rows in their next forward: nobody may start before every rank has finished its update
            flag = torch.zeros(1, device=s.flat.device)
            dist.all_reduce(flag)
        s.zero_grads()
        return grad_norm

    # ---------------------------------------------------------------- weights out
    def _full_named_parameters(self):
        """(native name, full tensor): sharded weights are all-gathered one at a time (a collective — every rank iterates)."""
        for n, p in self.model.named_parameters():
            sh = getattr(p, "_zero3", None)
            if sh is None and getattr(p, "_ep_full_shape", None) is not None:
                yield n, _gather_dim0(p.data, self.shard_group)
            else:
                yield n, (p.data if sh is None else _gather_rows(p.data, sh))

    def hf_named_tensors_for_save(self):
        from verl_b200.models.transformer import native_to_hf_tensors

        class _Lazy(dict):
            """Parameters by native name; a sharded entry is gathered when it is read and not kept."""

            def __init__(self, params):
                super().__init__(params)

            def __getitem__(self, k):
                p = super().__getitem__(k)
                sh = getattr(p, "_zero3", None)
                if sh is None and getattr(p, "_ep_full_shape", None) is not None:
                    return _gather_dim0(p.data, group)
                return p.data if sh is None else _gather_rows(p.data, sh)

        group = self.shard_group
        return native_to_hf_tensors(self.cfg, _Lazy(dict(self.model.named_parameters())))

    def get_per_tensor_param(self, **kwargs):
        return self.hf_named_tensors_for_save(), None

    def export_weights_source(self, file_path: Optional[str] = None) -> dict:
        raise NotImplementedError("zero3 mode hands weights over through get_per_tensor_param (collective gather)")

    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False, **kwargs):
        super().load_checkpoint(local_path, hdfs_path, del_local_after_load, **kwargs)
        if self.world > 1:
            dist.barrier()
