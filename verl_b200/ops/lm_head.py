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
