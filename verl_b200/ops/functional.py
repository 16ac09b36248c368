"""Differentiable front-ends of the sm_100a kernels.

Every op has two implementations behind one signature:

* **native** – bf16 CUDA tensors on a device where ``verl_b200/_C.so`` is loaded: the hand-written kernels;
* **reference** – plain PyTorch math in the input dtype (fp32 on CPU). It is the numerical oracle of the GPU tests
  and what the CPU/gloo configuration runs.

Weight gradients are written straight into ``param.main_grad`` (an fp32 view of the engine's flat gradient buffer)
when the parameter carries one, with the accumulation fused into the GEMM epilogue; autograd then sees ``None`` for
that input. This mirrors what FSDP's reduce dtype fp32 + gradient accumulation achieve in the reference
(``verl/workers/engine/fsdp/transformer_impl.py:396-405,695-726``) without extra copies.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _ext

__all__ = [
    "use_native", "gemm", "linear", "rmsnorm", "add_rmsnorm", "apply_rope_", "rope_tables", "swiglu", "embedding",
    "attention_varlen", "linear_logprob_entropy",
]


def use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and _ext.available()


# bf16 CUDA operands that the native kernels could not take (misaligned base / row stride): counted per reason and reported
# once each, so that a layout bug upstream shows up as a number instead of as a quietly slower step
fallback_counts: dict[str, int] = {}


def _note_fallback(reason: str, detail: str) -> None:
    n = fallback_counts.get(reason, 0)
    fallback_counts[reason] = n + 1
    if n == 0:
        import warnings

        warnings.warn(f"verl_b200.ops: {reason} runs on the PyTorch reference path ({detail}); further cases are only counted in "
                      "verl_b200.ops.functional.fallback_counts", RuntimeWarning, stacklevel=3)


# ------------------------------------------------------------------------------------------------ GEMM / linear
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, accumulate: bool = False, out_dtype: Optional[torch.dtype] = None,
         bn: int = 0) -> torch.Tensor:
    """out (+)= op(a) @ op(b)^T-style product. a: [M,K] (or [K,M] if a_mn); b: [N,K] (or [K,N] if b_mn)."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, device=a.device, dtype=out_dtype or a.dtype)
    if use_native(a) and _gemm_operand_ok(a) and _gemm_operand_ok(b):
        _ext.ops().gemm(a, b, out, bias, a_mn, b_mn, accumulate, bn)
        return out
    if use_native(a):
        _note_fallback("gemm with an operand the TMA descriptors cannot address",
                       f"a {tuple(a.shape)} strides {a.stride()} ptr%16={a.data_ptr() % 16}, b {tuple(b.shape)} strides {b.stride()} ptr%16={b.data_ptr() % 16}")
    A = a.t() if a_mn else a
    B = b if b_mn else b.t()
    r = (A.float() @ B.float()) if a.dtype != torch.float64 else A @ B
    if bias is not None:
        r = r + bias.float()
    if accumulate:
        out.add_(r.to(out.dtype))
    else:
        out.copy_(r.to(out.dtype))
    return out


def _gemm_operand_ok(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        ctx.bias_ref = bias
        return gemm(x, w, bias=bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                gemm(dy, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
            else:
                dw = gemm(dy, x, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            b = ctx.bias_ref
            bsum = dy.float().sum(0)
            mg = getattr(b, "main_grad", None)
            if mg is not None:
                mg.add_(bsum.to(mg.dtype))
            else:
                db = bsum.to(b.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ w.T + bias for 2-D x; weight gradient goes to ``w.main_grad`` when present."""
    if use_native(x) and x.dim() == 2:
        return _Linear.apply(x.contiguous(), w, bias)
    if getattr(w, "main_grad", None) is not None and torch.is_grad_enabled():
        return _Linear.apply(x, w, bias)
    return F.linear(x, w, bias)


# ------------------------------------------------------------------------------------------------ RMSNorm
def _rmsnorm_ref(x, w, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd).to(x.dtype) * w, rstd.squeeze(-1)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, _, rstd = _ext.ops().rmsnorm_fwd(x, None, w, eps, False)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        mg = getattr(w, "main_grad", None)
        dw_buf = mg if mg is not None else torch.zeros(w.numel(), device=w.device, dtype=torch.float32)
        dx = _ext.ops().rmsnorm_bwd(dy.contiguous(), x, w, rstd, None, dw_buf)
        return dx, (None if mg is not None else dw_buf.to(w.dtype)), None


class _AddRMSNorm(torch.autograd.Function):
    """r = x + residual; y = rmsnorm(r) * w. Returns (y, r); both inputs receive d(y→r) + dr."""

    @staticmethod
    def forward(ctx, x, residual, w, eps):
        y, r, rstd = _ext.ops().rmsnorm_fwd(x, residual, w, eps, True)
        ctx.save_for_backward(r, w, rstd)
        return y, r

    @staticmethod
    def backward(ctx, dy, dr):
        r, w, rstd = ctx.saved_tensors
        mg = getattr(w, "main_grad", None)
        dw_buf = mg if mg is not None else torch.zeros(w.numel(), device=w.device, dtype=torch.float32)
        dx = _ext.ops().rmsnorm_bwd(dy.contiguous(), r, w, rstd, dr.contiguous() if dr is not None else None, dw_buf)
        return dx, dx, (None if mg is not None else dw_buf.to(w.dtype)), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if use_native(x) and x.dim() == 2:
        return _RMSNorm.apply(x.contiguous(), w, eps)
    return _rmsnorm_ref(x, w, eps)[0]


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float):
    """Fused ``residual' = x + residual; y = rmsnorm(residual')``. Returns (y, residual')."""
    if use_native(x) and x.dim() == 2:
        return _AddRMSNorm.apply(x.contiguous(), residual.contiguous(), w, eps)
    r = x + residual
    return _rmsnorm_ref(r, w, eps)[0], r


# ------------------------------------------------------------------------------------------------ RoPE
_ROPE_CACHE: dict = {}


def scaled_inv_freq(dim: int, theta: float, scaling: Optional[dict], max_pos: int, device) -> tuple[torch.Tensor, float]:
    """Rotary frequencies under a Hugging Face ``rope_scaling`` / ``rope_parameters`` mapping, and the factor cos / sin are multiplied
    by (1 except for YaRN). Types: ``default`` / ``mrope`` (plain), ``linear`` (positions divided by ``factor``), ``llama3`` (long
    wavelengths divided by ``factor``, a smooth blend between ``low_freq_factor`` and ``high_freq_factor``), ``yarn`` (interpolated
    and extrapolated frequencies blended by a ramp between the ``beta_fast`` / ``beta_slow`` correction dimensions, attention factor
    ``0.1 ln(factor) + 1`` unless given). Reference behaviour: ``transformers.modeling_rope_utils`` as used by the reference's models."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    kind = str((scaling or {}).get("rope_type", (scaling or {}).get("type", "default")) or "default")
    if not scaling or kind in ("default", "mrope"):
        return inv, 1.0
    factor = float(scaling.get("factor", 1.0))
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        out = torch.where(wavelen > old / lo, inv / factor, inv)
        smooth = (old / wavelen - lo) / (hi - lo)
        blended = (1 - smooth) * out / factor + smooth * out
        medium = ~(wavelen < old / hi) & ~(wavelen > old / lo)
        return torch.where(medium, blended, out), 1.0
    if kind == "yarn":
        orig = float(scaling.get("original_max_position_embeddings") or max_pos)
        beta_fast, beta_slow = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)
        att = scaling.get("attention_factor")
        ms, ms_all = scaling.get("mscale"), scaling.get("mscale_all_dim")

        def get_mscale(scale, m=1.0):
            return 1.0 if scale <= 1 else 0.1 * float(m) * math.log(scale) + 1.0

        if att is None:
            att = get_mscale(factor, ms) / get_mscale(factor, ms_all) if ms and ms_all else get_mscale(factor)

        def corr_dim(n_rot):
            return (dim * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(theta))

        low, high = corr_dim(beta_fast), corr_dim(beta_slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
        extrap = 1 - ramp
        return (inv / factor) * (1 - extrap) + inv * extrap, float(att)
    raise NotImplementedError(f"rope scaling type {kind!r} is not supported")


def rope_tables(max_pos: int, dim: int, theta: float, device, scaling: Optional[dict] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables [max_pos, dim/2] (HF rotate-half convention: inv_freq = theta^(-2i/dim), modified by ``scaling``)."""
    key = (max_pos, dim, float(theta), str(device), tuple(sorted((k, str(v)) for k, v in (scaling or {}).items())))
    if key not in _ROPE_CACHE:
        inv, att = scaled_inv_freq(dim, theta, scaling, max_pos, device)
        ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
        _ROPE_CACHE[key] = ((ang.cos() * att).contiguous(), (ang.sin() * att).contiguous())
    return _ROPE_CACHE[key]


def _rope_ref(x, pos, cos, sin, nheads, D, sign):
    T = x.shape[0]
    xv = x[:, : nheads * D].reshape(T, nheads, D)
    c = cos[pos.long()][:, None, :].to(torch.float32)
    s = sin[pos.long()][:, None, :].to(torch.float32) * sign
    a, b = xv[..., : D // 2].float(), xv[..., D // 2 :].float()
    out = torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)
    return out.reshape(T, nheads * D)


class _Rope(torch.autograd.Function):
    """Rotates the first ``nheads*D`` columns of x ([T, ≥nheads*D]); remaining columns pass through."""

    @staticmethod
    def forward(ctx, x, pos, cos, sin, nheads, D):
        ctx.save_for_backward(pos, cos, sin)
        ctx.nheads, ctx.D = nheads, D
        if use_native(x):
            x = x.clone()
            _ext.ops().rope_(x, pos, cos, sin, nheads, D, 1.0)
            return x
        out = x.clone()
        out[:, : nheads * D] = _rope_ref(x, pos, cos, sin, nheads, D, 1.0)
        return out

    @staticmethod
    def backward(ctx, dy):
        pos, cos, sin = ctx.saved_tensors
        if use_native(dy):
            dx = dy.clone()
            _ext.ops().rope_(dx, pos, cos, sin, ctx.nheads, ctx.D, -1.0)
        else:
            dx = dy.clone()
            dx[:, : ctx.nheads * ctx.D] = _rope_ref(dy, pos, cos, sin, ctx.nheads, ctx.D, -1.0)
        return dx, None, None, None, None, None


def apply_rope_(qkv: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int, D: int):
    """Rotary embedding of the first ``n_rot_heads`` heads (q and k heads of a fused qkv row) — differentiable;
    under ``no_grad`` on the native path the rotation happens in place."""
    pos = pos.to(torch.int32)
    if not torch.is_grad_enabled() and use_native(qkv):
        _ext.ops().rope_(qkv, pos, cos, sin, n_rot_heads, D, 1.0)
        return qkv
    return _Rope.apply(qkv, pos, cos, sin, n_rot_heads, D)


# ------------------------------------------------------------------------------------------------ SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return _ext.ops().swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        return _ext.ops().swiglu_bwd(gu, dout.contiguous())


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """silu(gu[:, :I]) * gu[:, I:] for a fused gate|up activation."""
    if use_native(gu) and gu.dim() == 2:
        return _SwiGLU.apply(gu.contiguous())
    I = gu.shape[-1] // 2
    return F.silu(gu[..., :I]) * gu[..., I:]


# ------------------------------------------------------------------------------------------------ embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, w):
        ctx.save_for_backward(ids)
        ctx.w = w
        return w.index_select(0, ids)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.w
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            mg.index_add_(0, ids, dy.to(mg.dtype))
            return None, None
        dw = torch.zeros_like(w, dtype=torch.float32).index_add_(0, ids, dy.float()).to(w.dtype)
        return None, dw


def embedding(ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _Embedding.apply(ids, w)


# ------------------------------------------------------------------------------------------------ attention (packed varlen, causal, GQA)
def _attention_ref(q, k, v, cu_seqlens, scale):
    """q [T,Hq,D], k/v [T,Hkv,D]; loops over sequences (oracle / CPU path)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    out = torch.empty_like(q)
    cs = cu_seqlens.tolist()
    for b in range(len(cs) - 1):
        s, e = cs[b], cs[b + 1]
        if e == s:
            continue
        qb = q[s:e].transpose(0, 1).float()
        kb = k[s:e].transpose(0, 1).float().repeat_interleave(rep, dim=0)
        vb = v[s:e].transpose(0, 1).float().repeat_interleave(rep, dim=0)
        att = torch.matmul(qb, kb.transpose(1, 2)) * scale
        L = e - s
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        out[s:e] = torch.matmul(att, vb).transpose(0, 1).to(q.dtype)
    return out


def attention_varlen(qkv: torch.Tensor, cu_seqlens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     max_seqlen: int, cu_seqlens_cpu: Optional[torch.Tensor] = None, q_starts=None) -> torch.Tensor:
    """Causal self-attention over a packed batch. ``qkv`` is the fused projection output [T, (Hq+2Hkv)·D];
    returns [T, Hq·D]. ``q_starts`` (one per sequence): the rows before it only serve as keys/values, their outputs are
    undefined (the GPU kernels skip them, the reference path computes and the caller drops them)."""
    T = qkv.shape[0]
    scale = 1.0 / math.sqrt(head_dim)
    if use_native(qkv) and head_dim == 128:
        from .attention import flash_attention_varlen

        return flash_attention_varlen(qkv, cu_seqlens, n_heads, n_kv_heads, head_dim, max_seqlen, scale, cu_seqlens_cpu, q_starts)
    q, k, v = qkv.split([n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim], dim=-1)
    o = _attention_ref(q.reshape(T, n_heads, head_dim), k.reshape(T, n_kv_heads, head_dim),
                       v.reshape(T, n_kv_heads, head_dim), cu_seqlens if cu_seqlens_cpu is None else cu_seqlens_cpu, scale)
    return o.reshape(T, n_heads * head_dim)


# ------------------------------------------------------------------------------------------------ lm_head → logprob / entropy
def _linear_logprob_entropy_ref(h, w, labels, temperature, chunk=1024, need_entropy=True):
    logps, ents = [], []
    for i in range(0, h.shape[0], chunk):
        logits = (h[i : i + chunk].float() @ w.float().t()) / temperature
        lse = torch.logsumexp(logits, -1)
        logps.append(torch.gather(logits, -1, labels[i : i + chunk, None].long()).squeeze(-1) - lse)
        if need_entropy:
            ents.append(lse - (torch.softmax(logits, -1) * logits).sum(-1))
    lp = torch.cat(logps) if logps else h.new_zeros(0, dtype=torch.float32)
    en = torch.cat(ents) if need_entropy and ents else None
    return lp, en


def linear_logprob_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                           need_entropy: bool = True):
    """Per-token ``log_softmax(h @ w.T / τ)[label]`` and entropy without materialising [T, V] logits.

    Replaces the reference's Triton ``linear_cross_entropy`` (``verl/utils/kernel/linear_cross_entropy.py:38``) and the
    torch-chunked ``FusedLinearForPPO`` (``verl/utils/experimental/torch_functional.py:96``).
    """
    if use_native(h):
        from .lm_head import fused_linear_logprob

        return fused_linear_logprob(h, w, labels, temperature, need_entropy)
    if torch.is_grad_enabled() and (h.requires_grad or w.requires_grad):
        # differentiable chunked reference: checkpoint each chunk so [chunk, V] logits are never all alive
        from torch.utils.checkpoint import checkpoint

        logps, ents = [], []
        for i in range(0, h.shape[0], 512):
            def f(hc, wc, lc):
                lp, en = _linear_logprob_entropy_ref(hc, wc, lc, temperature, chunk=512, need_entropy=True)
                return lp, en
            lp, en = checkpoint(f, h[i : i + 512], w, labels[i : i + 512], use_reentrant=False)
            logps.append(lp)
            ents.append(en)
        return torch.cat(logps), (torch.cat(ents) if need_entropy else None)
    return _linear_logprob_entropy_ref(h, w, labels, temperature, need_entropy=need_entropy)
