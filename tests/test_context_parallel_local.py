"""Context-parallel attention without communication: one process plays every rank in turn on the rank-local part
(`cp_attention_local`) and the pieces must reproduce plain causal attention over the whole packed stream, outputs and
gradients, for the contiguous and the zig-zag placement. Sequence lengths are chosen so that slices start more than one
128-row tile into a sequence (the kernels then skip whole query tiles) and so that one sequence shows up in both chunks of a
zig-zag rank (duplicate K/V rows in the expanded layout)."""

from types import SimpleNamespace

import pytest
import torch

from verl_b200 import ops
from verl_b200.parallel.context_parallel import cp_attention_local, zigzag_permutation


def _run(device, dtype, head_dim, W, zigzag, lens, tol_o, tol_g):
    torch.manual_seed(0)
    cfg = SimpleNamespace(num_attention_heads=4, num_key_value_heads=2, head_dim=head_dim)
    q_size, kv_size = cfg.num_attention_heads * head_dim, 2 * cfg.num_key_value_heads * head_dim
    T = sum(lens)
    t_pad = T + (-T) % (2 * W)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens), 0)
    cu_full = cu if t_pad == T else torch.cat([cu, torch.tensor([t_pad], dtype=torch.int32)])      # padding = its own sequence
    x = (torch.randn(t_pad, q_size + kv_size, device=device) * 0.5).to(dtype).requires_grad_(True)
    g = (torch.randn(t_pad, q_size, device=device) * 0.1).to(dtype)

    ref = ops.attention_varlen(x, cu_full.to(device), cfg.num_attention_heads, cfg.num_key_value_heads, head_dim, max(lens + [t_pad - T]), cu_full)
    (gx_ref,) = torch.autograd.grad(ref, x, g)

    perm = (zigzag_permutation(t_pad, W) if zigzag else torch.arange(t_pad)).to(device)
    stream = x.index_select(0, perm)                 # rank-order concatenation of the local slices
    kv_all = stream[:, q_size:]
    tl = t_pad // W
    outs = [cp_attention_local(stream[r * tl:(r + 1) * tl, :q_size], kv_all, cu, cfg, W, r, zigzag) for r in range(W)]
    out = torch.cat(outs, 0)
    (gx,) = torch.autograd.grad(out, x, g.index_select(0, perm))
    if device == "cuda":
        from verl_b200.ops import _ext

        torch.cuda.synchronize()
        _ext.check_status("cp_attention_local")
    want = ref.index_select(0, perm)
    assert (out.float() - want.float()).abs().max().item() < tol_o
    # the padding rows attend among themselves in both formulations, so the comparison covers them too
    rel = ((gx.float() - gx_ref.float()).norm() / gx_ref.float().norm()).item()
    assert rel < tol_g, rel
    for name, sl in (("dq", slice(0, q_size)), ("dkv", slice(q_size, q_size + kv_size))):
        a, b = gx[:, sl].float(), gx_ref[:, sl].float()
        assert ((a - b).norm() / b.norm()).item() < tol_g, name


CASES = [(2, False, [700, 300, 150, 33]), (2, True, [700, 300, 150, 33]), (4, True, [700, 300, 150, 33]), (2, True, [160, 150, 140]),
         (3, True, [513, 77, 256]), (1, True, [300, 90])]


@pytest.mark.parametrize("W,zigzag,lens", CASES)
def test_cp_pieces_equal_full_attention_cpu(W, zigzag, lens):
    _run("cpu", torch.float32, 16, W, zigzag, lens, 1e-5, 1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("W,zigzag,lens", CASES)
def test_cp_pieces_equal_full_attention_gpu(W, zigzag, lens):
    _run("cuda", torch.bfloat16, 128, W, zigzag, lens, 0.03, 0.03)
