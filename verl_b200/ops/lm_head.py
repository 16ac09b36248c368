"""Autograd wrapper of the fused lm_head → log-prob / entropy kernels.

Forward: one tcgen05 GEMM whose epilogue reduces every 128×256 logits tile to softmax partials (no ``[T, V]`` tensor).
Backward: the vocabulary is walked in chunks; for each chunk the logits tile is recomputed and turned into dlogits in
the GEMM epilogue, then two GEMMs produce ``dh += dlogits·W_c`` and ``dW_c += dlogitsᵀ·h`` (the latter accumulated
straight into the fp32 main gradient).
"""

from __future__ import annotations

import torch

from . import _ext
from .functional import gemm

__all__ = ["fused_linear_logprob", "BWD_VOCAB_CHUNK"]

BWD_VOCAB_CHUNK = 16384


class _FusedLinearLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, temperature, need_entropy):
        labels = labels.to(torch.int64).contiguous()
        logp, ent, lse = _ext.ops().lmhead_logprob_fwd(h, w, labels, 1.0 / temperature)
        ctx.save_for_backward(h, w, labels, lse, ent)
        ctx.temperature = temperature
        ctx.need_entropy = need_entropy
        ctx.mark_non_differentiable(lse)
        return logp, ent, lse

    @staticmethod
    def backward(ctx, g_lp, g_ent, _g_lse):
        h, w, labels, lse, ent = ctx.saved_tensors
        M, K = h.shape
        V = w.shape[0]
        inv_t = 1.0 / ctx.temperature
        g_lp = (g_lp if g_lp is not None else torch.zeros_like(lse)).float().contiguous()
        g_ent_c = g_ent.float().contiguous() if (g_ent is not None and ctx.need_entropy) else None
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh_acc = torch.zeros(M, K, dtype=torch.float32, device=h.device) if need_dh else None
        mg = getattr(w, "main_grad", None)
        dw = None
        if need_dw and mg is None:
            dw = torch.zeros(V, K, dtype=torch.float32, device=h.device)
        dw_target = mg if mg is not None else dw
        chunk = min(BWD_VOCAB_CHUNK, V)
        buf = torch.empty(M, chunk, dtype=torch.bfloat16, device=h.device)
        for c0 in range(0, V, chunk):
            vc = min(chunk, V - c0)
            w_c = w[c0 : c0 + vc]
            d = buf[:, :vc]
            _ext.ops().lmhead_dlogits(h, w_c, labels, inv_t, c0, lse, ent, g_lp, g_ent_c, d)
            if need_dh:
                gemm(d, w_c, b_mn=True, out=dh_acc, accumulate=True)
            if need_dw:
                gemm(d, h, a_mn=True, b_mn=True, out=dw_target[c0 : c0 + vc], accumulate=True)
        dh = dh_acc.to(h.dtype) if need_dh else None
        return dh, (dw.to(w.dtype) if dw is not None else None), None, None, None


def fused_linear_logprob(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                         need_entropy: bool = True):
    if h.shape[0] == 0:
        z = torch.zeros(0, dtype=torch.float32, device=h.device)
        return z, (z.clone() if need_entropy else None)
    logp, ent, _ = _FusedLinearLogprob.apply(h.contiguous(), w, labels, float(temperature), bool(need_entropy))
    return logp, (ent if need_entropy else None)


# ---------------------------------------------------------------------------------------------------------------------
# Vocabulary-parallel version: each tensor-parallel rank owns rows [voff, voff + V_local) of the output matrix.
# Forward runs the same fused kernel on the local slice and merges (lse, label logit, E[x]) across ranks with ONE
# all-gather of a [3, T] tensor; backward feeds the GLOBAL lse / entropy to the dlogits kernel, whose formula then is
# exactly the gradient of the global softmax restricted to the local columns. Reference: three all-reduces around the
# Triton epilogue (verl/utils/kernel/kernels.py:708-740) and verl/utils/megatron/tensor_parallel.py:109-210.
def _local_stats(h, w, labels_local, inv_t, native):
    """(lse, label_logit (0 where the label is not local), E_local[x]) in fp32 for the local vocabulary slice."""
    V = w.shape[0]
    mine = (labels_local >= 0) & (labels_local < V)
    if native:
        lp, ent, lse = _ext.ops().lmhead_logprob_fwd(h, w, torch.where(mine, labels_local, torch.full_like(labels_local, -1)), inv_t)
        lab = torch.where(mine, lp + lse, torch.zeros_like(lse))
        return lse, lab, lse - ent
    lses, labs, exs = [], [], []
    for i in range(0, h.shape[0], 1024):
        x = (h[i : i + 1024].float() @ w.float().t()) * inv_t
        l = torch.logsumexp(x, -1)
        p = torch.exp(x - l[:, None])
        m = mine[i : i + 1024]
        idx = torch.where(m, labels_local[i : i + 1024], torch.zeros_like(labels_local[i : i + 1024]))
        labs.append(torch.where(m, x.gather(1, idx[:, None])[:, 0], torch.zeros_like(l)))
        lses.append(l)
        exs.append((p * x).sum(-1))
    return torch.cat(lses), torch.cat(labs), torch.cat(exs)


class _VocabParallelLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, temperature, need_entropy, group, voff):
        import torch.distributed as dist

        native = h.is_cuda and _ext.available() and h.dtype == torch.bfloat16
        labels = labels.to(torch.int64).contiguous()
        inv_t = 1.0 / temperature
        lse_r, lab_r, ex_r = _local_stats(h, w, labels - voff, inv_t, native)
        W = dist.get_world_size(group)
        mine = torch.stack([lse_r, lab_r, ex_r]).float().contiguous()
        flat = torch.empty(W * 3, mine.shape[1], dtype=mine.dtype, device=mine.device)
        dist.all_gather_into_tensor(flat, mine, group=group)
        allv = flat.view(W, 3, -1)
        lse = torch.logsumexp(allv[:, 0], 0)
        label_logit = allv[:, 1].sum(0)
        ex = (torch.exp(allv[:, 0] - lse[None]) * allv[:, 2]).sum(0)
        logp, ent = label_logit - lse, lse - ex
        ctx.save_for_backward(h, w, labels, lse, ent)
        ctx.cfg = (temperature, need_entropy, voff, native)
        return logp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        h, w, labels, lse, ent = ctx.saved_tensors
        temperature, need_entropy, voff, native = ctx.cfg
        inv_t = 1.0 / temperature
        M, K = h.shape
        V = w.shape[0]
        g_lp = (g_lp if g_lp is not None else torch.zeros_like(lse)).float().contiguous()
        g_ent_c = g_ent.float().contiguous() if (g_ent is not None and need_entropy) else None
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh_acc = torch.zeros(M, K, dtype=torch.float32, device=h.device) if need_dh else None
        mg = getattr(w, "main_grad", None)
        dw = torch.zeros(V, K, dtype=torch.float32, device=h.device) if (need_dw and mg is None) else None
        dw_target = mg if mg is not None else dw
        chunk = min(BWD_VOCAB_CHUNK if native else 4096, V)
        buf = torch.empty(M, chunk, dtype=torch.bfloat16, device=h.device) if native else None
        for c0 in range(0, V, chunk):
            vc = min(chunk, V - c0)
            w_c = w[c0 : c0 + vc]
            if native:
                d = buf[:, :vc]
                _ext.ops().lmhead_dlogits(h, w_c, labels, inv_t, voff + c0, lse, ent, g_lp, g_ent_c, d)
                if need_dh:
                    gemm(d, w_c, b_mn=True, out=dh_acc, accumulate=True)
                if need_dw:
                    gemm(d, h, a_mn=True, b_mn=True, out=dw_target[c0 : c0 + vc], accumulate=True)
            else:
                x = (h.float() @ w_c.float().t()) * inv_t
                p = torch.exp(x - lse[:, None])
                onehot = (labels[:, None] - (voff + c0)) == torch.arange(vc, device=h.device)[None]
                d = g_lp[:, None] * (onehot.float() - p)
                if g_ent_c is not None:
                    d = d - g_ent_c[:, None] * p * (x - lse[:, None] + ent[:, None])
                d = d * inv_t
                if need_dh:
                    dh_acc += d @ w_c.float()
                if need_dw:
                    dw_target[c0 : c0 + vc] += d.t() @ h.float()
        dh = dh_acc.to(h.dtype) if need_dh else None
        return dh, (dw.to(w.dtype) if dw is not None else None), None, None, None, None, None


def vocab_parallel_logprob(h: torch.Tensor, w_local: torch.Tensor, labels: torch.Tensor, temperature: float, need_entropy: bool,
                           group, vocab_offset: int):
    """``h`` must be the same on every rank of ``group`` (pass it through ``copy_to_tp`` first so its gradient is summed)."""
    logp, ent = _VocabParallelLogprob.apply(h.contiguous(), w_local, labels, float(temperature), bool(need_entropy), group, int(vocab_offset))
    return logp, (ent if need_entropy else None)
