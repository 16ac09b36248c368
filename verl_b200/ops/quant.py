"""Low-precision casts: block-wise fp8 (e4m3) for rollout weights / activations and NVFP4 fake quantisation for QAT.

Each function runs the sm_100a kernel on CUDA bf16 inputs and an equivalent PyTorch formulation elsewhere (which is also
the oracle of the GPU tests). Reference: ``verl/utils/kernel/fp8_kernel.py:53-260`` (scale convention: the stored
``scale`` is what you MULTIPLY by to dequantise, i.e. ``weight_scale_inv`` in vLLM terms) and ``verl/utils/qat/linear.py:
42-330`` (``fp4_fake_quant_weight``, ``STEFP4QuantTriton``, ``QATLinear``).
"""

from __future__ import annotations

import torch

from . import _ext
from .functional import use_native

__all__ = ["blockwise_cast_to_fp8", "act_cast_to_fp8", "dequant_blockwise_fp8", "rowwise_cast_to_fp8", "fp8_gemm", "fp8_linear", "FP8Linear", "fp8_block_gemm", "fp8_block_linear", "fp4_fake_quant", "fp4_fake_quant_ste", "QATLinear",
           "FP8_MAX", "FP4_MAX"]

FP8_MAX, FP4_MAX = 448.0, 6.0


def _blockwise_ref(x: torch.Tensor, bm: int, bn: int):
    M, N = x.shape
    pm, pn = (-M) % bm, (-N) % bn
    xp = torch.nn.functional.pad(x.float(), (0, pn, 0, pm))
    blocks = xp.reshape((M + pm) // bm, bm, (N + pn) // bn, bn)
    s = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10) / FP8_MAX
    q = (blocks * (1.0 / s)[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).reshape(M + pm, N + pn)[:M, :N]
    return q.to(torch.float8_e4m3fn), s


def blockwise_cast_to_fp8(x: torch.Tensor, block_size=(128, 128)):
    """``x [M, N]`` → ``(fp8 [M, N], scale [ceil(M/bm), ceil(N/bn)])`` with ``scale = max(absmax, 1e-10) / 448``."""
    assert x.dim() == 2
    if tuple(block_size) == (128, 128) and use_native(x):
        return _ext.ops().fp8_block_cast(x if x.stride(1) == 1 else x.contiguous())
    return _blockwise_ref(x, int(block_size[0]), int(block_size[1]))


def act_cast_to_fp8(x: torch.Tensor):
    """Dynamic per-token 1×128 group quantisation of activations: ``(fp8 [M, K], scale [M, ceil(K/128)])``."""
    assert x.dim() == 2
    if use_native(x) and x.shape[1] % 4 == 0:
        return _ext.ops().fp8_act_cast(x if x.stride(1) == 1 else x.contiguous())
    return _blockwise_ref(x, 1, 128)


def rowwise_cast_to_fp8(x: torch.Tensor):
    """One scale per row: ``(fp8 [M, K], scale [M])``, ``scale = max(absmax(row), 1e-12) / 448``. Per-token for activations,
    per-output-channel for ``[N, K]`` weights — the scales then factor out of the K sum and the GEMM applies them in its
    epilogue (``fp8_gemm``)."""
    assert x.dim() == 2
    if use_native(x) and x.shape[1] % 8 == 0:
        return _ext.ops().fp8_row_cast(x if x.stride(1) == 1 else x.contiguous())
    s = x.float().abs().amax(-1).clamp_min(1e-12) / FP8_MAX
    return (x.float() / s[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s


def fp8_gemm(a8: torch.Tensor, b8: torch.Tensor, a_scale: torch.Tensor = None, b_scale: torch.Tensor = None, bias: torch.Tensor = None,
             out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``diag(a_scale) · (a8 @ b8ᵀ) · diag(b_scale) (+ bias)`` with e4m3 operands ``a8 [M, K]``, ``b8 [N, K]``.

    On sm_100a this is one tcgen05 ``kind::f8f6f4`` kernel on SM pairs (256×256 tiles, fp32 accumulation in TMEM, scales and
    bias in the epilogue); elsewhere the operands are dequantised and multiplied in fp32."""
    if a8.is_cuda and _ext.available() and a8.shape[1] % 16 == 0 and out_dtype in (torch.bfloat16, torch.float32):
        a8 = a8 if a8.stride(1) == 1 and a8.stride(0) % 16 == 0 else a8.contiguous()
        b8 = b8 if b8.stride(1) == 1 and b8.stride(0) % 16 == 0 else b8.contiguous()
        return _ext.ops().gemm_fp8(a8, b8, a_scale, b_scale, bias, out_dtype == torch.float32)
    y = a8.float() @ b8.float().t()
    if a_scale is not None:
        y = y * a_scale[:, None] * b_scale[None, :]
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)


def fp8_linear(x: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor, bias: torch.Tensor = None) -> torch.Tensor:
    """W8A8 linear for inference: ``x`` (bf16, any leading shape) is quantised per token on the fly, ``w8 / w_scale`` come from
    ``rowwise_cast_to_fp8(weight)``."""
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    a8, a_s = rowwise_cast_to_fp8(x2)
    return fp8_gemm(a8, w8, a_s, w_scale, bias, x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16).reshape(*shp[:-1], w8.shape[0])


def fp8_block_gemm(a8: torch.Tensor, a_scale: torch.Tensor, b8: torch.Tensor, b_scale: torch.Tensor, bias: torch.Tensor = None,
                   out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Block-scaled e4m3 GEMM: ``a8 [M, K]`` with 1×128 scales ``a_scale [M, ⌈K/128⌉]`` (``act_cast_to_fp8``), ``b8 [N, K]`` with
    128×128 scales ``b_scale [⌈N/128⌉, ⌈K/128⌉]`` (``blockwise_cast_to_fp8``) — the layout fp8 rollout weights are shipped in.
    sm_100a: tcgen05 ``kind::f8f6f4`` partial products per K block, promoted with their scales in registers."""
    if a8.is_cuda and _ext.available() and a8.shape[1] % 16 == 0 and out_dtype in (torch.bfloat16, torch.float32):
        a8 = a8 if a8.stride(1) == 1 and a8.stride(0) % 16 == 0 else a8.contiguous()
        b8 = b8 if b8.stride(1) == 1 and b8.stride(0) % 16 == 0 else b8.contiguous()
        return _ext.ops().gemm_fp8_block(a8, a_scale.contiguous(), b8, b_scale.contiguous(), bias, out_dtype == torch.float32)
    M, K = a8.shape
    N = b8.shape[0]
    a = a8.float() * a_scale.repeat_interleave(128, 1)[:, :K]
    b = b8.float() * b_scale.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    y = a @ b.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)


def fp8_block_linear(x: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor, bias: torch.Tensor = None) -> torch.Tensor:
    """Linear layer on block-quantised weights (``blockwise_cast_to_fp8(weight)``) with 1×128 dynamic activation scales."""
    shp = x.shape
    a8, a_s = act_cast_to_fp8(x.reshape(-1, shp[-1]))
    return fp8_block_gemm(a8, a_s, w8, w_scale, bias, x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16).reshape(*shp[:-1], w8.shape[0])


class FP8Linear(torch.nn.Module):
    """Frozen linear layer with per-output-channel e4m3 weights (built from a bf16 weight), dynamic per-token activations."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor = None):
        super().__init__()
        w8, ws = rowwise_cast_to_fp8(weight.detach())
        self.register_buffer("weight", w8)
        self.register_buffer("weight_scale", ws)
        self.register_buffer("bias", bias.detach().clone() if bias is not None else None)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return fp8_linear(x, self.weight, self.weight_scale, self.bias)


def dequant_blockwise_fp8(q: torch.Tensor, scale: torch.Tensor, block_size=(128, 128), dtype=torch.bfloat16) -> torch.Tensor:
    M, N = q.shape
    s = scale.repeat_interleave(block_size[0], 0)[:M].repeat_interleave(block_size[1], 1)[:, :N]
    return (q.float() * s).to(dtype)


_E2M1_EDGES = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _fp4_ref(x: torch.Tensor, global_amax: torch.Tensor, block: int = 16) -> torch.Tensor:
    shape = x.shape
    g = x.float().reshape(-1, block)
    gs = global_amax.float() / (FP4_MAX * FP8_MAX)
    gs_safe = torch.where(gs > 0, gs, torch.full_like(gs, 1e-12))
    sc = (g.abs().amax(-1, keepdim=True) / (FP4_MAX * gs_safe)).clamp(max=FP8_MAX)
    sc = sc.to(torch.float8_e4m3fn).float() * gs
    sc = torch.where(sc >= 1e-5, sc, torch.ones_like(sc))
    a = g.abs() / sc
    q = torch.zeros_like(a)
    # round half to even on the E2M1 grid: ties at .25, 1.25, 2.5, 5 go down; ties at .75, 1.75, 3.5 go up
    for k, (edge, val) in enumerate(zip(_E2M1_EDGES, _E2M1_VALUES[1:])):
        up_on_tie = k % 2 == 1
        q = torch.where((a >= edge) if up_on_tie else (a > edge), torch.full_like(a, val), q)
    return (torch.sign(g) * q * sc).reshape(shape).to(x.dtype)


def fp4_fake_quant(x: torch.Tensor, global_amax: torch.Tensor = None, block_size: int = 16) -> torch.Tensor:
    """Quantise-dequantise to NVFP4 (E2M1 values, e4m3 group scales relative to ``global_amax / (6·448)``)."""
    if global_amax is None:
        global_amax = x.detach().abs().max().float()
    global_amax = global_amax.reshape(1).float()
    if block_size == 16 and use_native(x) and x.shape[-1] % 16 == 0:
        return _ext.ops().fp4_fake_quant(x.contiguous(), global_amax.to(x.device))
    return _fp4_ref(x, global_amax.to(x.device), block_size)


class _FP4STE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, global_amax, block_size):
        return fp4_fake_quant(x, global_amax, block_size)

    @staticmethod
    def backward(ctx, g):
        return g, None, None


def fp4_fake_quant_ste(x: torch.Tensor, global_amax: torch.Tensor = None, block_size: int = 16) -> torch.Tensor:
    """Fake quantisation with a straight-through gradient (quantisation-aware training)."""
    return _FP4STE.apply(x, global_amax, block_size)


class QATLinear(torch.nn.Module):
    """Linear layer whose weight (and, in ``w4a4`` mode, input) passes through NVFP4 fake quantisation in forward.

    ``weight_amax`` is the global amax used for the group scales; it is initialised from the weight on first use and can
    be synchronised across ranks with ``sync_amax(group)`` (an all-reduce MAX, as the reference does for FSDP shards).
    """

    def __init__(self, weight: torch.nn.Parameter, bias=None, mode: str = "w4a16", block_size: int = 16):
        super().__init__()
        assert mode in ("w4a16", "w4a4")
        self.weight, self.bias, self.mode, self.block_size = weight, bias, mode, block_size
        self.register_buffer("weight_amax", torch.full((1,), -1.0, dtype=torch.float32, device=weight.device))

    @torch.no_grad()
    def sync_amax(self, group=None):
        import torch.distributed as dist

        amax = self.weight.detach().abs().max().float().reshape(1)
        if dist.is_initialized() and (group is not None or dist.get_world_size() > 1):
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
        self.weight_amax.copy_(amax)

    def forward(self, x):
        if float(self.weight_amax) < 0:
            self.sync_amax()
        w = fp4_fake_quant_ste(self.weight, self.weight_amax, self.block_size)
        if self.mode == "w4a4":
            x = fp4_fake_quant_ste(x, None, self.block_size)
        return torch.nn.functional.linear(x, w, self.bias)
