"""sm_100a quantisation casts and weight-delta kernels against their PyTorch formulations."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fp8_block_cast_matches_reference():
    from verl_b200.ops.quant import _blockwise_ref, act_cast_to_fp8, blockwise_cast_to_fp8

    for M, N in ((512, 1024), (300, 200), (129, 136)):
        x = (torch.randn(M, N, device="cuda") * 2).bfloat16()
        q, s = blockwise_cast_to_fp8(x)
        qr, sr = _blockwise_ref(x, 128, 128)
        torch.testing.assert_close(s, sr, rtol=1e-6, atol=0)
        assert (q.float() - qr.float()).abs().max() <= 32.0 and (q.float() != qr.float()).float().mean() < 1e-3   # at most rounding ties
        qa, sa = act_cast_to_fp8(x) if N % 4 == 0 else (None, None)
        if qa is not None:
            qar, sar = _blockwise_ref(x, 1, 128)
            torch.testing.assert_close(sa, sar, rtol=1e-6, atol=0)
            assert (qa.float() != qar.float()).float().mean() < 1e-3


def test_fp4_fake_quant_matches_reference():
    from verl_b200.ops.quant import _fp4_ref, fp4_fake_quant

    x = (torch.randn(257, 512, device="cuda") * 0.05).bfloat16()
    amax = x.abs().max().float().reshape(1)
    y = fp4_fake_quant(x, amax)
    ref = _fp4_ref(x, amax)
    assert (y.float() != ref.float()).float().mean() < 1e-3
    torch.testing.assert_close(y.float(), ref.float(), rtol=0, atol=float(amax) * 0.2)


def test_delta_compact_and_apply_kernels():
    from verl_b200.checkpoint_engine import delta_apply, delta_compact

    n = 8 * 1024 * 1024 + 4096
    old = torch.randn(n, device="cuda").bfloat16()
    new = old.clone()
    idx = torch.randperm(n, device="cuda")[:50000]
    new[idx] = (new[idx].float() + 1.0).bfloat16()
    changed = (new.view(torch.int16) != old.view(torch.int16)).sum().item()
    snap, recv = old.clone(), old.clone()
    count, pos, val = delta_compact(new, snap)
    assert count == changed and torch.equal(snap, new)
    assert torch.equal(torch.sort(pos.long())[0], torch.nonzero(new.view(torch.int16) != old.view(torch.int16)).reshape(-1))
    delta_apply(recv, pos, val)
    assert torch.equal(recv, new)
    # overflow of the pair buffers is reported through the count
    snap2 = old.clone()
    count2, pos2, _ = delta_compact(new, snap2, cap=1000)
    assert count2 == changed and pos2.numel() == 1000


def test_reshard_gather_and_requant_from_row_shards():
    """Two 'trainer shards' (here both in this GPU's memory) are gathered into a rollout row range and block-quantised."""
    from verl_b200.checkpoint_engine.reshard import gather_rows, gather_rows_fp8
    from verl_b200.ops.quant import _blockwise_ref

    full = (torch.randn(768, 520, device="cuda") * 1.5).bfloat16()
    shards = [full[:384].contiguous(), full[384:].contiguous()]
    ptrs = [s.data_ptr() for s in shards]
    got = gather_rows(ptrs, 384, 520, 256, 300, full)
    assert torch.equal(got, full[256:556])
    q, sc, keep = gather_rows_fp8(ptrs, 384, 520, 256, 300, full, keep_bf16=True)
    qr, sr = _blockwise_ref(full[256:556], 128, 128)
    torch.testing.assert_close(sc, sr, rtol=1e-6, atol=0)
    assert torch.equal(keep, full[256:556]) and (q.float() != qr.float()).float().mean() < 1e-3


def test_reshard_into_parameter_slices_rows_and_columns():
    """The in-place gather behind the actor -> rollout weight hand-off, with the 'trainer ranks' emulated by two buffers of this
    GPU: a tensor-parallel rollout slice is either a set of row ranges (column-parallel layers: q | k | v blocks) or a column
    range of every row (row-parallel layers). Results are bitwise equal to slicing the gathered matrix; memory outside the
    destination view stays untouched."""
    from verl_b200.checkpoint_engine.reshard import gather_rows_into

    torch.manual_seed(3)
    N, K, W = 1536, 1024, 2
    full = torch.randn(N, K, device="cuda").bfloat16()
    shards = [full[r * (N // W):(r + 1) * (N // W)].contiguous() for r in range(W)]
    ptrs = torch.tensor([s.data_ptr() for s in shards], dtype=torch.int64)
    # column-parallel: rollout rank 1 of 2 owns the second half of each of three row blocks (sizes 1024 | 256 | 256)
    segs, tp, tp_rank = [1024, 256, 256], 2, 1
    dst = torch.full((sum(n // tp for n in segs) + 16, K), 7.0, device="cuda", dtype=torch.bfloat16)      # 16 guard rows
    off = doff = 0
    for n in segs:
        per = n // tp
        gather_rows_into(ptrs, N // W, K, off + tp_rank * per, dst[doff:doff + per])
        off += n
        doff += per
    want = torch.cat([full[0:1024][512:], full[1024:1280][128:], full[1280:1536][128:]])
    assert torch.equal(dst[:doff], want) and bool((dst[doff:] == 7.0).all())
    # row-parallel: rollout rank 1 of 2 owns columns [512, 1024) of every row; the destination is a column window of a wider buffer
    wide = torch.full((N, K // 2 + 16), 7.0, device="cuda", dtype=torch.bfloat16)
    gather_rows_into(ptrs, N // W, K, 0, wide[:, 8:8 + K // 2], col_begin=K // 2)
    assert torch.equal(wide[:, 8:8 + K // 2], full[:, K // 2:]) and bool((wide[:, :8] == 7.0).all()) and bool((wide[:, 8 + K // 2:] == 7.0).all())


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(512, 768, 1024), (300, 520, 2064), (2048, 4096, 4096), (17, 40, 144)])
def test_fp8_gemm_matches_dequantised_reference(M, N, K):
    """e4m3 tcgen05 GEMM with row/column scales vs the fp32 product of the dequantised operands (ragged edges included)."""
    from verl_b200.ops import _ext
    from verl_b200.ops.quant import fp8_gemm, fp8_linear, rowwise_cast_to_fp8

    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    a8, sa = rowwise_cast_to_fp8(x)
    b8, sb = rowwise_cast_to_fp8(w)
    # the cast kernel against its definition
    sa_ref = x.float().abs().amax(-1).clamp_min(1e-12) / 448.0
    assert torch.allclose(sa, sa_ref, rtol=1e-6)
    want8 = (x.float() * (1.0 / sa_ref)[:, None]).to(torch.float8_e4m3fn).float()
    diff = (a8.float() - want8).abs()
    # the kernel's reciprocal may differ from torch's in the last bit: a value on a rounding boundary can land one e4m3 step off
    assert (diff > 0).float().mean().item() < 2e-3 and (diff <= 0.13 * want8.abs() + 2 ** -9).all()
    ref = (a8.float() * sa[:, None]) @ (b8.float() * sb[:, None]).t() + bias.float()
    y = fp8_gemm(a8, b8, sa, sb, bias)
    y32 = fp8_gemm(a8, b8, sa, sb, bias, out_dtype=torch.float32)
    assert (y32 - ref).abs().max() <= 1e-3 * ref.abs().max()
    assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    raw = fp8_gemm(a8, b8, out_dtype=torch.float32)                      # unscaled product
    assert (raw - a8.float() @ b8.float().t()).abs().max() <= 1e-3 * raw.abs().max()
    # W8A8 linear is close to the bf16 linear (quantisation error only)
    z = fp8_linear(x, b8, sb, bias)
    full = x.float() @ w.float().t() + bias.float()
    assert ((z.float() - full).norm() / full.norm()).item() < 0.06
    torch.cuda.synchronize()
    _ext.check_status("fp8 gemm")


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (300, 520, 2064), (1024, 3584, 4096), (17, 40, 144)])
def test_fp8_block_scaled_gemm(M, N, K):
    """Block-scaled e4m3 GEMM (1x128 activation scales, 128x128 weight scales) vs the fp32 product of the dequantised operands."""
    from verl_b200.ops import _ext
    from verl_b200.ops.quant import act_cast_to_fp8, blockwise_cast_to_fp8, fp8_block_gemm, fp8_block_linear

    torch.manual_seed(M + N + K)
    # rows and blocks of very different magnitude: wrong scale indexing would show immediately
    x = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 1, M, device="cuda")[:, None]).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05 * (1 + torch.arange(N, device="cuda")[:, None] // 128) * (1 + torch.arange(K, device="cuda")[None, :] // 128)).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    a8, sa = act_cast_to_fp8(x)
    b8, sb = blockwise_cast_to_fp8(w)
    a_deq = a8.float() * sa.repeat_interleave(128, 1)[:, :K]
    b_deq = b8.float() * sb.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    ref = a_deq @ b_deq.t() + bias.float()
    y32 = fp8_block_gemm(a8, sa, b8, sb, bias, out_dtype=torch.float32)
    y = fp8_block_gemm(a8, sa, b8, sb, bias)
    torch.cuda.synchronize()
    _ext.check_status("fp8 block gemm")
    assert (y32 - ref).abs().max() <= 2e-3 * ref.abs().max(), ((y32 - ref).abs().max().item(), ref.abs().max().item())
    assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    z = fp8_block_linear(x, b8, sb, bias)
    full = x.float() @ w.float().t() + bias.float()
    assert ((z.float() - full).norm() / full.norm()).item() < 0.06
