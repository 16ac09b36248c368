"""MoE routing, permutation and the padded grouped layout (CPU); the grouped GEMM kernels are checked in the GPU suite."""

import torch

from verl_b200.ops.moe import moe_forward, padded_layout, permute_tokens, route_topk, unpermute_tokens


def test_router_replay_and_permutation_roundtrip():
    torch.manual_seed(0)
    T, H, E, k = 37, 16, 8, 2
    x = torch.randn(T, H)
    logits = torch.randn(T, E)
    w, idx, probs = route_topk(logits, k, True)
    assert torch.allclose(w.sum(-1), torch.ones(T)) and (idx == probs.topk(k).indices).all()
    forced = idx.flip(-1).clone()
    forced[0] = -1
    w2, idx2, _ = route_topk(logits, k, True, forced)
    assert (idx2[1:] == forced[1:]).all() and (idx2[0] == idx[0]).all()
    xp, order, counts = permute_tokens(x, idx, E)
    assert counts.sum() == T * k and torch.equal(xp, x[order // k])
    y = unpermute_tokens(xp, order, w, T)
    assert torch.allclose(y, x * w.sum(-1, keepdim=True), atol=1e-6)


def test_padded_layout_tables():
    counts = torch.tensor([3, 0, 130, 128, 1])
    n = int(counts.sum())
    dest, R, blk, rng = padded_layout(counts, n, block=128)
    assert R % 128 == 0 and R >= 128 * 5 and dest.shape == (n,)
    assert rng.tolist() == [[0, 1], [1, 1], [1, 3], [3, 4], [4, 5]]
    assert blk[:5].tolist() == [0, 2, 2, 3, 4] and (blk[5:] == -1).all()
    assert dest[:3].tolist() == [0, 1, 2] and dest[3] == 128 and dest[3 + 130] == 384 and dest[-1] == 512
    assert len(set(dest.tolist())) == n


def test_moe_forward_matches_dense_reference():
    torch.manual_seed(1)
    T, H, I, E, k = 24, 32, 48, 4, 2
    x = torch.randn(T, H, requires_grad=True)
    router, gu, dn = torch.randn(E, H), torch.randn(E, 2 * I, H) * 0.1, torch.randn(E, H, I) * 0.1
    y, idx = moe_forward(x, router, gu, dn, k, True)
    w, idx2, _ = route_topk(x @ router.t(), k, True)
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(idx2[t, j])
            g, u = (x[t] @ gu[e].t()).split(I)
            ref[t] += w[t, j] * ((torch.nn.functional.silu(g) * u) @ dn[e].t())
    assert torch.equal(idx, idx2) and torch.allclose(y, ref, atol=1e-4)
    y.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
