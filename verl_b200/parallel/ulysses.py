"""Ulysses sequence parallelism: tokens are sharded over the SP group everywhere except inside attention, where an
all-to-all trades the sequence shard for a head shard (each rank sees the full sequence for ``heads / sp`` heads).

Parity target: ``verl/utils/ulysses.py`` (SeqAllToAll :169-196, gather_seq_scatter_heads :66, gather_heads_scatter_seq
:90, pad/slice :282-334, gather_outputs_and_unpad :247-280) and the attention hook
``verl/models/transformers/monkey_patch.py:87-155`` (KV-head replication when ``sp > n_kv_heads``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

__all__ = ["SeqAllToAll", "gather_seq_scatter_heads", "gather_heads_scatter_seq", "Gather", "ulysses_pad_and_slice_inputs",
           "gather_outputs_and_unpad", "ulysses_attention", "validate_ulysses_config", "FusedUlysses", "fused_ulysses_available"]


def _a2a(x: torch.Tensor, scatter_dim: int, gather_dim: int, group) -> torch.Tensor:
    ws = dist.get_world_size(group)
    if ws == 1:
        return x
    parts = [t.contiguous() for t in torch.tensor_split(x, ws, dim=scatter_dim)]
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: every rank gathers everyone's pieces and keeps the ones addressed to it (CPU test path)
        mine = torch.stack(parts)
        allp = [torch.empty_like(mine) for _ in range(ws)]
        dist.all_gather(allp, mine, group=group)
        me = dist.get_rank(group)
        outs = [allp[r][me] for r in range(ws)]
    else:
        outs = [torch.empty_like(parts[0]) for _ in range(ws)]
        dist.all_to_all(outs, parts, group=group)
    return torch.cat(outs, dim=gather_dim).contiguous()


class SeqAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, x, scatter_dim, gather_dim):
        ctx.group, ctx.scatter_dim, ctx.gather_dim = group, scatter_dim, gather_dim
        return _a2a(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, g):
        return None, _a2a(g, ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None


def gather_seq_scatter_heads(x: torch.Tensor, seq_dim: int, head_dim: int, group, unpadded_dim_size: int = 0) -> torch.Tensor:
    """[.., T/sp, .., H, ..] → [.., T, .., H/sp, ..]"""
    if group is None or dist.get_world_size(group) == 1:
        return x
    x = SeqAllToAll.apply(group, x, head_dim, seq_dim)
    if unpadded_dim_size and unpadded_dim_size % dist.get_world_size(group) != 0:
        x = x.narrow(seq_dim, 0, unpadded_dim_size)
    return x


def gather_heads_scatter_seq(x: torch.Tensor, head_dim: int, seq_dim: int, group) -> torch.Tensor:
    """[.., T, .., H/sp, ..] → [.., T/sp, .., H, ..]"""
    if group is None or dist.get_world_size(group) == 1:
        return x
    sp = dist.get_world_size(group)
    pad = (-x.shape[seq_dim]) % sp
    if pad:
        shape = list(x.shape)
        shape[seq_dim] = pad
        x = torch.cat([x, x.new_zeros(shape)], dim=seq_dim)
    return SeqAllToAll.apply(group, x, seq_dim, head_dim)


class Gather(torch.autograd.Function):
    """all-gather along ``dim`` forward; backward keeps this rank's slice (scaled by sp when ``grad_scaler``)."""

    @staticmethod
    def forward(ctx, group, x, dim, grad_scaler=True):
        ctx.group, ctx.dim, ctx.grad_scaler = group, dim, grad_scaler
        ws, ctx.rank = dist.get_world_size(group), dist.get_rank(group)
        ctx.part = x.shape[dim]
        outs = [torch.empty_like(x) for _ in range(ws)]
        dist.all_gather(outs, x.contiguous(), group=group)
        return torch.cat(outs, dim=dim)

    @staticmethod
    def backward(ctx, g):
        if ctx.grad_scaler:
            g = g * dist.get_world_size(ctx.group)
        return None, g.narrow(ctx.dim, ctx.rank * ctx.part, ctx.part).contiguous(), None, None


def ulysses_pad_and_slice_inputs(input_ids: torch.Tensor, position_ids: Optional[torch.Tensor], sp_size: int, sp_rank: int, dim: int = -1):
    """Pad the packed token axis to a multiple of ``sp_size`` and keep this rank's contiguous slice.
    Returns (ids_slice, pos_slice, pad_size)."""
    T = input_ids.shape[dim]
    pad = (-T) % sp_size
    if pad:
        input_ids = torch.nn.functional.pad(input_ids, (0, pad), value=0)
        if position_ids is not None:
            extra = torch.arange(pad, device=position_ids.device, dtype=position_ids.dtype)
            position_ids = torch.cat([position_ids, extra], dim=dim)
    part = (T + pad) // sp_size
    sl = slice(sp_rank * part, (sp_rank + 1) * part)
    return input_ids[..., sl], (position_ids[..., sl] if position_ids is not None else None), pad


def gather_outputs_and_unpad(x: torch.Tensor, gather_dim: int, unpad_dim: Optional[int] = None, padding_size: int = 0, grad_scaler: bool = True, group=None):
    if group is None or dist.get_world_size(group) == 1:
        return x
    x = Gather.apply(group, x, gather_dim, grad_scaler)
    if unpad_dim is not None and padding_size:
        x = x.narrow(unpad_dim, 0, x.shape[unpad_dim] - padding_size)
    return x


def validate_ulysses_config(num_heads: int, num_kv_heads: int, sp: int):
    assert num_heads % sp == 0, f"num_attention_heads ({num_heads}) must be divisible by ulysses sp size ({sp})"
    assert num_kv_heads % sp == 0 or sp % num_kv_heads == 0, f"kv heads ({num_kv_heads}) and sp size ({sp}) must divide one another"


def ulysses_attention(qkv: torch.Tensor, pb, cfg, group) -> torch.Tensor:
    """Attention on a sequence-sharded fused qkv [T/sp, (Hq+2Hkv)·D]: a2a to [T, (Hq+2Hkv')/sp·D], full-sequence
    attention on the local heads, a2a back to [T/sp, Hq·D]. ``pb`` describes the *global* packed batch."""
    from verl_b200 import ops

    sp = dist.get_world_size(group)
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    validate_ulysses_config(Hq, Hkv, sp)
    Tl = qkv.shape[0]
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    q, k, v = q.reshape(Tl, Hq, D), k.reshape(Tl, Hkv, D), v.reshape(Tl, Hkv, D)
    if Hkv < sp:                       # replicate kv heads so that every rank owns at least one
        rep = sp // Hkv
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    q = gather_seq_scatter_heads(q, 0, 1, group)
    k = gather_seq_scatter_heads(k, 0, 1, group)
    v = gather_seq_scatter_heads(v, 0, 1, group)
    T = int(pb.cu_seqlens_cpu[-1])
    hq_l, hkv_l = q.shape[1], k.shape[1]
    fused = torch.cat([q[:T].reshape(T, -1), k[:T].reshape(T, -1), v[:T].reshape(T, -1)], dim=-1)
    o = ops.attention_varlen(fused, pb.cu_seqlens, hq_l, hkv_l, D, pb.max_seqlen, pb.cu_seqlens_cpu).reshape(T, hq_l, D)
    o = gather_heads_scatter_seq(o, 1, 0, group)
    return o[:Tl].reshape(Tl, Hq * D)


# ---------------------------------------------------------------------------------------------------------------------
# Fused path: the two all-to-alls disappear into the projections around attention.
#   * QKV projection: the GEMM epilogue writes every output head straight into the memory of the rank that owns that head
#     (rows = this rank's token slice) — ``gemm_head_scatter``;
#   * output projection: the GEMM's A operand is read tile by tile from the ranks that hold the corresponding heads
#     (K axis split over ranks) — ``gemm_kseg``.
# Backward mirrors them: d(attention output) = (dY @ W_o) routed to the head owners by the same scatter epilogue, and
# dX = gather_over_ranks(dQKV) @ W_qkv through the same K-segmented gather (W_qkv's rows permuted into rank-major order); the
# gathered dQKV left in the staging buffer feeds the weight gradient. Only the re-gather of the attention output for the
# output projection's weight gradient still uses an NCCL all-to-all.
def fused_ulysses_available(x: torch.Tensor, cfg, sp: int) -> bool:
    import os

    from verl_b200.ops import _ext

    return (x.is_cuda and x.dtype == torch.bfloat16 and _ext.available() and os.environ.get("VERL_B200_COMM", "native") == "native"
            and cfg.head_dim % 32 == 0 and cfg.num_attention_heads % sp == 0 and cfg.num_key_value_heads % sp == 0
            and (cfg.num_attention_heads // sp * cfg.head_dim) % 64 == 0)


class FusedUlysses:
    """Symmetric staging buffers and head routing tables of one SP group (shared by all layers of a model)."""

    def __init__(self, group, host_group, cfg, max_tokens: int):
        from verl_b200.ops import _ext
        from verl_b200.parallel.symm_mem import SymmetricBuffer

        self.group, self.cfg, self.ops = group, cfg, _ext.ops()
        self._host_group = host_group
        self.sp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        self.hq_l, self.hkv_l = Hq // self.sp, Hkv // self.sp
        self.Cl, self.Kl = (self.hq_l + 2 * self.hkv_l) * D, self.hq_l * D
        self.max_tokens = max_tokens
        self.qkv_buf = SymmetricBuffer(max_tokens * self.Cl * 2, group, host_group)
        self.o_buf = SymmetricBuffer(max_tokens * self.Kl * 2, group, host_group)
        rank_of, slot_of = [], []
        for h in range(Hq):
            rank_of.append(h // self.hq_l)
            slot_of.append(h % self.hq_l)
        for base in (self.hq_l, self.hq_l + self.hkv_l):          # k heads, then v heads
            for j in range(Hkv):
                rank_of.append(j // self.hkv_l)
                slot_of.append(base + j % self.hkv_l)
        self.head_rank = torch.tensor(rank_of, dtype=torch.int32)
        self.head_slot = torch.tensor(slot_of, dtype=torch.int32)
        dev = torch.device("cuda", torch.cuda.current_device())
        tl_max = -(-max_tokens // self.sp // 128) * 128 + 128
        self.o_stage = torch.empty(tl_max * Hq * D, dtype=torch.bfloat16, device=dev)     # peers' head slices of the local token rows
        self.o_flags = torch.zeros((tl_max // 128) * self.sp + 8, dtype=torch.int32, device=dev)
        self.o_epoch = 0
        self.fused_backward = True
        # backward: gradient buffers the peers write (d attention output) or read (d qkv), staging of the gathered d qkv, and the
        # order in which rank-major columns [rank][q | k | v heads of that rank] appear among the rows of the qkv weight
        self.do_buf = self.dqkv_buf = None
        self.tl_max = tl_max
        self.q_rank = self.head_rank[:Hq].clone()
        self.q_slot = self.head_slot[:Hq].clone()
        order = sorted(range(Hq + 2 * Hkv), key=lambda h: (rank_of[h], slot_of[h]))
        self.row_perm = torch.tensor([h * D + i for h in order for i in range(D)], dtype=torch.long, device=dev)
        self.col_unperm = torch.argsort(self.row_perm)

    def _backward_buffers(self, host_group=None):
        if self.do_buf is None:
            from verl_b200.parallel.symm_mem import SymmetricBuffer

            dev = self.o_stage.device
            self.do_buf = SymmetricBuffer(self.max_tokens * self.Kl * 2, self.group, self._host_group)
            self.dqkv_buf = SymmetricBuffer(self.max_tokens * self.Cl * 2, self.group, self._host_group)
            self.g_stage = torch.empty(self.tl_max * self.sp * self.Cl, dtype=torch.bfloat16, device=dev)
            self.g_flags = torch.zeros((self.tl_max // 128) * self.sp + 8, dtype=torch.int32, device=dev)
            self.g_epoch = 0

    def o_backward(self, g, w_o, Tl: int):
        """d(attention output of the local heads, all tokens) [Tp, Kl] from dY [Tl, hidden]: (dY @ W_o) with head h sent to rank
        h // hq_l by the GEMM epilogue."""
        self._backward_buffers()
        Tp = Tl * self.sp
        self.do_buf.barrier()             # every rank has copied the previous layer's result out of its buffer
        self.ops.gemm_head_scatter(g, w_o, None, self.do_buf.table(), self.Kl, self.rank * Tl, self.cfg.head_dim, self.q_rank, self.q_slot, True)
        self.do_buf.barrier()
        return self.do_buf.tensor(torch.bfloat16, Tp * self.Kl).view(Tp, self.Kl).clone()

    def qkv_backward(self, g, w, Tl: int):
        """dX [Tl, hidden] and dQKV in sequence layout [Tl, N] (weight-row order) from g [Tp, Cl] (local heads, all tokens)."""
        self._backward_buffers()
        Tp, N = Tl * self.sp, self.sp * self.Cl
        self.dqkv_buf.tensor(torch.bfloat16, Tp * self.Cl).view(Tp, self.Cl).copy_(g)
        self.dqkv_buf.barrier()
        dx = torch.empty(Tl, w.shape[1], dtype=torch.bfloat16, device=g.device)
        self.g_epoch += 1
        w_rank_major = w.index_select(0, self.row_perm)          # rows in the order the ranks hold the columns of d qkv
        self.ops.gemm_kseg(self.dqkv_buf.table(), self.Cl, Tp, self.rank * Tl, w_rank_major, dx, None, self.rank, self.g_stage, self.g_flags,
                           self.g_epoch, True)
        Tl_pad = -(-Tl // 128) * 128
        dy_rm = self.g_stage[: Tl_pad * N].view(Tl_pad, N)[:Tl]
        dy_rm[:, self.rank * self.Cl:(self.rank + 1) * self.Cl].copy_(g[self.rank * Tl:(self.rank + 1) * Tl])     # own columns were read in place
        self.dqkv_buf.barrier()           # the peers have finished reading this rank's gradient rows
        return dx, dy_rm.index_select(1, self.col_unperm)

    def qkv_forward(self, x_shard, w, bias):
        Tl = x_shard.shape[0]
        Tp = Tl * self.sp
        assert Tp <= self.max_tokens, f"{Tp} tokens exceed the staging buffers ({self.max_tokens})"
        self.ops.gemm_head_scatter(x_shard, w, bias, self.qkv_buf.table(), self.Cl, self.rank * Tl, self.cfg.head_dim, self.head_rank, self.head_slot)
        self.qkv_buf.barrier()
        return self.qkv_buf.tensor(torch.bfloat16, Tp * self.Cl).view(Tp, self.Cl).clone()

    def o_forward(self, o_local, w_o, Tl: int):
        Tp = Tl * self.sp
        self.o_buf.tensor(torch.bfloat16, Tp * self.Kl).view(Tp, self.Kl).copy_(o_local)
        self.o_buf.barrier()
        out = torch.empty(Tl, w_o.shape[0], dtype=torch.bfloat16, device=o_local.device)
        self.o_epoch += 1
        self.ops.gemm_kseg(self.o_buf.table(), self.Kl, Tp, self.rank * Tl, w_o, out, None, self.rank, self.o_stage, self.o_flags, self.o_epoch)
        return out

    # ---- layout conversions used by the (unfused) backward passes
    def heads_to_seq(self, t_local):
        """[Tp, n_l·D] (local heads, all tokens) → [Tl, n·D] (all heads, local tokens)."""
        D = self.cfg.head_dim
        Tp = t_local.shape[0]
        return _a2a(t_local.reshape(Tp, -1, D), 0, 1, self.group).reshape(Tp // self.sp, -1)

    def seq_to_heads(self, t_shard):
        """[Tl, n·D] → [Tp, n_l·D]."""
        D = self.cfg.head_dim
        Tl = t_shard.shape[0]
        return _a2a(t_shard.reshape(Tl, -1, D), 1, 0, self.group).reshape(Tl * self.sp, -1)


class _FusedQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, fu: FusedUlysses):
        ctx.save_for_backward(x, w)
        ctx.fu, ctx.bias_ref = fu, bias
        return fu.qkv_forward(x.contiguous(), w, bias)

    @staticmethod
    def backward(ctx, g):
        from verl_b200.ops.functional import gemm

        x, w = ctx.saved_tensors
        fu = ctx.fu
        if ctx.needs_input_grad[0] and fu.fused_backward and x.shape[0] * fu.sp <= fu.max_tokens:
            dx, dy = fu.qkv_backward(g.contiguous(), w, x.shape[0])
        else:
            q_w, k_w = fu.hq_l * fu.cfg.head_dim, fu.hkv_l * fu.cfg.head_dim
            gq, gk, gv = g.split([q_w, k_w, k_w], dim=-1)
            dy = torch.cat([fu.heads_to_seq(gq.contiguous()), fu.heads_to_seq(gk.contiguous()), fu.heads_to_seq(gv.contiguous())], dim=-1).contiguous()
            dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                gemm(dy, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
            else:
                dw = gemm(dy, x, a_mn=True, b_mn=True)
        b = ctx.bias_ref
        if b is not None and ctx.needs_input_grad[2]:
            bsum = dy.float().sum(0)
            mg = getattr(b, "main_grad", None)
            if mg is not None:
                mg.add_(bsum.to(mg.dtype))
            else:
                db = bsum.to(b.dtype)
        return dx, dw, db, None


class _FusedOProj(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o_local, w_o, fu: FusedUlysses, Tl: int):
        ctx.save_for_backward(o_local, w_o)
        ctx.fu = fu
        return fu.o_forward(o_local.contiguous(), w_o, Tl)

    @staticmethod
    def backward(ctx, g):
        from verl_b200.ops.functional import gemm

        o_local, w_o = ctx.saved_tensors
        fu = ctx.fu
        g = g.contiguous()
        if ctx.needs_input_grad[0] and fu.fused_backward:
            do_local = fu.o_backward(g, w_o, g.shape[0])
        else:
            do_local = fu.seq_to_heads(gemm(g, w_o, b_mn=True)) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            o_shard = fu.heads_to_seq(o_local).contiguous()
            mg = getattr(w_o, "main_grad", None)
            if mg is not None:
                gemm(g, o_shard, a_mn=True, b_mn=True, out=mg, accumulate=True)
            else:
                dw = gemm(g, o_shard, a_mn=True, b_mn=True)
        return do_local, dw, None, None


def fused_ulysses_attention_block(x_shard, attn_mod, pb, cfg, fu: FusedUlysses, cos, sin):
    """QKV projection → (a2a) → RoPE → attention on local heads → (a2a) → output projection, for one layer.
    ``pb.global_position_ids`` holds the padded positions of ALL tokens of the micro-batch."""
    from verl_b200 import ops

    Tl = x_shard.shape[0]
    T = int(pb.cu_seqlens_cpu[-1])
    fused = _FusedQKV.apply(x_shard, attn_mod.qkv_proj, attn_mod.qkv_bias, fu)
    fused = ops.apply_rope_(fused, pb.global_position_ids, cos, sin, fu.hq_l + fu.hkv_l, cfg.head_dim)
    o = ops.attention_varlen(fused[:T], pb.cu_seqlens, fu.hq_l, fu.hkv_l, cfg.head_dim, pb.max_seqlen, pb.cu_seqlens_cpu)
    if T < Tl * fu.sp:
        o = torch.cat([o, o.new_zeros(Tl * fu.sp - T, o.shape[1])], 0)
    return _FusedOProj.apply(o, attn_mod.o_proj, fu, Tl)
