"""sm_100a kernels against plain PyTorch fp32 references of the same ops (run with ``-m gpu`` on a B200)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def o():
    from verl_b200.ops import _ext

    _ext.load()
    return _ext.ops()


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


def status_ok(o):
    torch.cuda.synchronize()
    return int(o.take_status()) == 0


@pytest.mark.parametrize("M,N,K,a_mn,b_mn,bn,f32,acc,bias", [
    (128, 256, 64, False, False, 256, False, False, False),
    (256, 512, 256, False, False, 128, False, False, False),
    (256, 512, 256, False, False, 64, False, False, False),
    (256, 512, 256, False, False, 32, False, False, False),
    (300, 520, 200, False, False, 0, False, False, True),      # ragged M, N, K tails + bias
    (384, 392, 264, False, True, 0, False, False, False),      # input-gradient layout
    (392, 520, 1000, True, True, 0, True, True, False),        # weight-gradient layout, fp32 accumulate
    (256, 256, 512, True, False, 128, False, False, False),
    (4096, 3584, 3584, False, False, 0, False, False, False),
])
def test_gemm_layouts(o, M, N, K, a_mn, b_mn, bn, f32, acc, bias):
    dev = "cuda"
    torch.manual_seed(0)
    a = (torch.randn(K, M, device=dev) if a_mn else torch.randn(M, K, device=dev)).bfloat16()
    b = (torch.randn(K, N, device=dev) if b_mn else torch.randn(N, K, device=dev)).bfloat16()
    bs = torch.randn(N, device=dev).bfloat16() if bias else None
    out = (torch.randn(M, N, device=dev) if acc else torch.empty(M, N, device=dev)).to(torch.float32 if f32 else torch.bfloat16)
    base = out.float().clone() if acc else 0
    o.gemm(a, b, out, bs, a_mn, b_mn, acc, bn)
    assert status_ok(o)
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    ref = A @ B + base + (bs.float() if bias else 0)
    assert rel(out, ref) < (1e-5 if f32 else 8e-3)


@pytest.mark.parametrize("M,N,K,a_mn,b_mn,f32,acc,bias", [
    (512, 1024, 256, False, False, False, False, False),       # two row blocks x two column tiles, exact fit
    (520, 1160, 328, False, False, False, False, True),        # ragged M, N, K tails + bias
    (768, 1544, 512, False, True, False, False, False),        # input-gradient layout
    (776, 1032, 1096, True, True, True, True, False),          # weight-gradient layout: fp32 reduce-add into the output
    (512, 1024, 512, True, True, True, False, False),          # fp32 store
    (1024, 1024, 320, True, False, False, False, False),
    (4096, 4608, 3584, False, False, False, False, True),      # several tiles per pair: accumulator hand-over between tiles
    (2304, 19456, 512, False, False, False, False, False),     # more tiles than SM pairs, grouped tile order
    (3584, 3584, 8192, True, True, True, True, False),         # 98 tiles on 74 pairs: K slices that reduce-add into the output
])
def test_gemm_pair512_with_canaries(o, M, N, K, a_mn, b_mn, f32, acc, bias):
    """The 256 x 512-tile kernel (bn = 514) against an fp32 matmul. The output is a window inside a larger buffer whose
    guard rows and columns must come back untouched: the TMA-store epilogue clips at the tensor-map extents."""
    dev = "cuda"
    torch.manual_seed(1)
    a = (torch.randn(K, M, device=dev) if a_mn else torch.randn(M, K, device=dev)).bfloat16()
    b = (torch.randn(K, N, device=dev) if b_mn else torch.randn(N, K, device=dev)).bfloat16()
    bs = torch.randn(N, device=dev).bfloat16() if bias else None
    dt = torch.float32 if f32 else torch.bfloat16
    G = 8                                            # guard: 8 rows above/below, 8 columns left/right (keeps 16-byte alignment)
    big = torch.full((M + 2 * G, N + 2 * G), 7.0, device=dev, dtype=dt)
    out = big[G:G + M, G:G + N]
    if acc:
        out.copy_(torch.randn(M, N, device=dev))
    base = out.float().clone() if acc else 0
    o.gemm(a, b, out, bs, a_mn, b_mn, acc, 514)
    assert status_ok(o)
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    ref = A @ B + base + (bs.float() if bias else 0)
    assert rel(out, ref) < (5e-5 if f32 else 8e-3)
    guard = big.clone()
    guard[G:G + M, G:G + N] = 7.0
    assert bool((guard == 7.0).all()), "the kernel wrote outside its output window"


def test_elementwise_ops(o):
    from verl_b200.ops import functional as Fn

    dev = "cuda"
    torch.manual_seed(0)
    T, H, I = 300, 3584, 1024
    x = torch.randn(T, H, device=dev).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
    r = torch.randn(T, H, device=dev).bfloat16()
    assert rel(Fn.rmsnorm(x, w, 1e-6), Fn._rmsnorm_ref(x, w, 1e-6)[0]) < 1e-2
    y2, r2 = Fn.add_rmsnorm(x, r, w, 1e-6)
    assert rel(y2, Fn._rmsnorm_ref(x + r, w, 1e-6)[0]) < 1e-2 and torch.equal(r2, x + r)
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    Fn.rmsnorm(xg, wg, 1e-6).float().pow(2).sum().backward()
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr).pow(2).sum().backward()
    assert rel(xg.grad, xr.grad) < 2e-2 and rel(wg.grad, wr.grad) < 1e-2
    gu = torch.randn(T, 2 * I, device=dev).bfloat16().requires_grad_(True)
    out = Fn.swiglu(gu)
    out.float().sum().backward()
    gr = gu.detach().float().requires_grad_(True)
    ref = torch.nn.functional.silu(gr[:, :I]) * gr[:, I:]
    ref.sum().backward()
    assert rel(out, ref) < 1e-2 and rel(gu.grad, gr.grad) < 1e-2
    cos, sin = Fn.rope_tables(4096, 128, 1e6, dev)
    qkv = torch.randn(T, 36 * 128, device=dev).bfloat16()
    pos = torch.randint(0, 4096, (T,), device=dev, dtype=torch.int32)
    want = qkv.clone()
    want[:, : 32 * 128] = Fn._rope_ref(qkv, pos, cos, sin, 32, 128, 1.0)
    got = qkv.clone()
    o.rope_(got, pos, cos, sin, 32, 128, 1.0)
    assert rel(got, want) < 5e-3
    o.rope_(got, pos, cos, sin, 32, 128, -1.0)            # inverse rotation restores the input (backward path)
    assert rel(got, qkv) < 2e-2
    assert status_ok(o)


def test_adamw_and_norm(o):
    dev = "cuda"
    torch.manual_seed(0)
    n = 1000003
    p32, g = torch.randn(n, device=dev), torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    pr = p32.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pr], lr=1e-3, weight_decay=0.01)
    for step in (1, 2):
        pr.grad = g.clone()
        opt.step()
        o.adamw_(p32, m, v, g, p16, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, torch.tensor([1.0, 0.0, 0.0, 0.0], device=dev))
    assert (p32 - pr.detach()).abs().max().item() < 1e-5 and rel(p16, pr.detach()) < 5e-3
    before = p32.clone()
    o.adamw_(p32, m, v, g, p16, 1e-3, 0.9, 0.999, 1e-8, 0.01, 3, torch.tensor([1.0, 1.0, 0.0, 0.0], device=dev))   # skip flag
    assert torch.equal(before, p32)
    ss = torch.zeros(1, device=dev)
    o.sqnorm_(g, ss)
    assert abs(ss.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-5
    sc = torch.zeros(4, device=dev)
    o.clip_coef_(ss, 1.0, sc)
    assert abs(sc[2].item() - math.sqrt(ss.item())) < 1e-2 and abs(sc[0].item() - 1.0 / (math.sqrt(ss.item()) + 1e-6)) < 1e-6


@pytest.mark.parametrize("lens,Hq,Hkv", [([128], 1, 1), ([200, 77, 400], 4, 2), ([1000, 5, 129, 256], 14, 2)])
def test_attention_varlen_fwd_bwd(o, lens, Hq, Hkv):
    from verl_b200 import ops
    from verl_b200.ops import functional as Fn

    dev, D, T = "cuda", 128, sum(lens)
    torch.manual_seed(0)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    qkv = (0.5 * torch.randn(T, (Hq + 2 * Hkv) * D, device=dev)).bfloat16().requires_grad_(True)
    out = ops.attention_varlen(qkv, cu.to(dev), Hq, Hkv, D, max(lens), cu)
    dout = torch.randn_like(out)
    out.backward(dout)
    assert status_ok(o)
    q2 = qkv.detach().float().requires_grad_(True)
    q, k, v = q2.split([Hq * D, Hkv * D, Hkv * D], -1)
    ref = Fn._attention_ref(q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D), cu, 1 / math.sqrt(D)).reshape(T, Hq * D)
    ref.backward(dout.float())
    assert rel(out, ref) < 1e-2 and rel(qkv.grad, q2.grad) < 1.5e-2


@pytest.mark.parametrize("lens,q_starts", [([640, 300], [256, 0]), ([1000, 77, 515], [700, 40, 384]), ([384], [383])])
def test_attention_varlen_with_key_only_prefix_rows(o, lens, q_starts):
    """Context-parallel form: rows before q_starts[s] carry only keys/values. Their query tiles are skipped in forward and
    backward; the remaining rows and all K/V gradients equal the plain causal attention."""
    from verl_b200 import ops
    from verl_b200.ops import functional as Fn

    dev, D, Hq, Hkv, T = "cuda", 128, 4, 2, sum(lens)
    torch.manual_seed(1)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    live = torch.cat([torch.arange(L) >= qs for L, qs in zip(lens, q_starts)]).to(dev)
    base = (0.5 * torch.randn(T, (Hq + 2 * Hkv) * D, device=dev)).bfloat16()
    base[:, : Hq * D] *= live[:, None]                     # no queries before q_start
    qkv = base.clone().requires_grad_(True)
    out = ops.attention_varlen(qkv, cu.to(dev), Hq, Hkv, D, max(lens), cu, q_starts=tuple(q_starts))
    dout = torch.randn_like(out) * live[:, None]
    torch.where(live[:, None], out, torch.zeros_like(out)).backward(dout)
    assert status_ok(o)
    q2 = base.float().requires_grad_(True)
    q, k, v = q2.split([Hq * D, Hkv * D, Hkv * D], -1)
    ref = Fn._attention_ref(q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D), cu, 1 / math.sqrt(D)).reshape(T, Hq * D)
    ref.backward(dout.float())
    assert rel(out[live], ref[live]) < 1e-2
    g, gr = qkv.grad.float(), q2.grad
    assert torch.isfinite(g[:, Hq * D:]).all() and rel(g[:, Hq * D:], gr[:, Hq * D:]) < 1.5e-2       # dK, dV of every row
    assert rel(g[live][:, : Hq * D], gr[live][:, : Hq * D]) < 1.5e-2                                    # dQ of the live rows


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("B,Hq,Hkv,lens,splits", [(3, 28, 4, [5, 200, 512], 1), (3, 28, 4, [5, 200, 512], 2), (2, 8, 8, [64, 129], 1), (2, 28, 4, [0, 300], 4),
                                                  (4, 32, 2, [1, 127, 128, 400], 1)])
def test_paged_decode_attention(o, B, Hq, Hkv, lens, splits, impl):
    from verl_b200.ops.attention import paged_decode_attention, paged_decode_attention_ref

    dev, D, nb, maxb = "cuda", 128, 64, 8
    torch.manual_seed(0)
    cache = (0.5 * torch.randn(nb, 2, Hkv, 64, D, device=dev)).bfloat16()
    bt = torch.stack([torch.randperm(nb)[:maxb] for _ in range(B)]).to(torch.int32).to(dev)
    kl = torch.tensor(lens, dtype=torch.int32, device=dev)
    q = (0.5 * torch.randn(B, Hq * D, device=dev)).bfloat16()
    ws = torch.empty(B * Hq * splits * 130, device=dev) if splits > 1 else None
    out = paged_decode_attention(q, cache, bt, kl, 1 / math.sqrt(D), splits, max(lens), ws, impl=impl)
    assert status_ok(o)
    assert rel(out, paged_decode_attention_ref(q, cache, bt, kl, 1 / math.sqrt(D))) < 1.5e-2


@pytest.mark.parametrize("M,V,K,temp", [(300, 1000, 256, 1.0), (1000, 20000, 512, 0.7), (130, 152064, 128, 1.0)])
def test_fused_lm_head_logprob_entropy(o, M, V, K, temp):
    from verl_b200 import ops

    dev = "cuda"
    torch.manual_seed(0)
    h = (0.5 * torch.randn(M, K, device=dev)).bfloat16().requires_grad_(True)
    w = (0.05 * torch.randn(V, K, device=dev)).bfloat16().requires_grad_(True)
    lab = torch.randint(0, V, (M,), device=dev)
    lp, en = ops.linear_logprob_entropy(h, w, lab, temp, True)
    glp, gen = torch.randn(M, device=dev), torch.randn(M, device=dev)
    (lp * glp + en * gen).sum().backward()
    assert status_ok(o)
    h2, w2 = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    logits = (h2 @ w2.t()) / temp
    lse = torch.logsumexp(logits, -1)
    lpr = logits.gather(-1, lab[:, None]).squeeze(-1) - lse
    enr = lse - (torch.softmax(logits, -1) * logits).sum(-1)
    (lpr * glp + enr * gen).sum().backward()
    assert (lp - lpr).abs().max().item() < 2e-3 and (en - enr).abs().max().item() < 2e-3
    assert rel(h.grad, h2.grad) < 1.5e-2 and rel(w.grad, w2.grad) < 1.5e-2


def test_sampling_kernel_distribution_and_filters(o):
    dev = "cuda"
    B, V = 512, 1000
    logits = torch.zeros(B, V, device=dev)
    logits[:, :4] = torch.tensor([3.0, 2.0, 1.0, 0.0], device=dev)
    logits[:, 4:] = -20.0
    rng = torch.tensor([123, 0], dtype=torch.int64, device=dev)
    tok = torch.empty(B, dtype=torch.int64, device=dev)
    lp = torch.empty(B, dtype=torch.float32, device=dev)
    counts = torch.zeros(4)
    for step in range(8):
        rng[1] = step
        o.sample(logits, 1.0, -1, 1.0, rng, None, tok, lp)
        counts += torch.bincount(tok.cpu(), minlength=V)[:4].float()
    p = torch.softmax(torch.tensor([3.0, 2.0, 1.0, 0.0]), 0)
    assert (counts / counts.sum() - p).abs().max() < 0.03
    want_lp = torch.log_softmax(logits[0].float(), 0)[tok[0]]
    assert abs(lp[0].item() - want_lp.item()) < 1e-3
    o.sample(logits, 1.0, 2, 1.0, rng, None, tok, lp)
    assert set(tok.tolist()) <= {0, 1}
    o.sample(logits, 1.0, -1, 0.6, rng, None, tok, lp)     # p0 = 0.64 >= 0.6 -> only the top token survives
    assert set(tok.tolist()) == {0}
    o.sample(logits.bfloat16(), 0.0, -1, 1.0, rng, None, tok, lp)
    assert set(tok.tolist()) == {0}


def test_kv_cache_write(o):
    dev, Hq, Hkv, D, T = "cuda", 4, 2, 128, 37
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
    cache = torch.zeros(8, 2, Hkv, 64, D, device=dev, dtype=torch.bfloat16)
    slots = torch.randperm(8 * 64, device=dev)[:T]
    slots[3] = -1
    o.kv_cache_write(qkv, slots, cache, Hq, Hkv)
    torch.cuda.synchronize()
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    for t in (0, 1, 10, 36):
        b, off = int(slots[t]) // 64, int(slots[t]) % 64
        assert torch.equal(cache[b, 0, :, off], k[t]) and torch.equal(cache[b, 1, :, off], v[t])
    assert cache.abs().sum(dim=(1, 2, 3, 4)).count_nonzero() <= 8


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_pair_cta_group_2(a_mn, b_mn):
    """256 x 256 tiles computed by SM pairs (tcgen05.mma.cta_group::2) against an fp32 matmul, ragged edges included."""
    from verl_b200.ops import _ext

    o = _ext.ops()
    torch.manual_seed(0)
    for M, N, K in ((512, 512, 256), (1000, 776, 328), (2304, 1536, 1024)):
        a = (torch.randn(K, M, device="cuda") if a_mn else torch.randn(M, K, device="cuda")).bfloat16()
        b = (torch.randn(K, N, device="cuda") if b_mn else torch.randn(N, K, device="cuda")).bfloat16()
        ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        o.gemm(a, b, out, None, a_mn, b_mn, False, 512)
        _ext.check_status("gemm_pair")
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=0.35)
        acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
        bias = torch.randn(N, device="cuda").bfloat16()
        o.gemm(a, b, acc, bias, a_mn, b_mn, True, 512)
        _ext.check_status("gemm_pair accumulate")
        torch.testing.assert_close(acc, ref + 1.0 + bias.float()[None], rtol=1e-3, atol=2e-2)


@pytest.mark.parametrize("M,N,K", [(256, 3584, 18944), (200, 1000, 4160), (512, 37888, 3584), (130, 256, 520)])
def test_gemm_pair_split_k_for_decode_shapes(M, N, K):
    """Decode-sized GEMMs on SM pairs with K slices (fp32 partial tiles + reduce pass) against an fp32 matmul."""
    from verl_b200.ops import _ext

    o = _ext.ops()
    torch.manual_seed(M + N)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    o.gemm(a, b, out, bias, False, False, False, 513)
    _ext.check_status("gemm_pair split-k")
    torch.testing.assert_close(out.float(), ref + bias.float()[None], rtol=2e-2, atol=0.2)
    acc = torch.full((M, N), 2.0, device="cuda", dtype=torch.float32)
    o.gemm(a, b, acc, None, False, False, True, 513)
    _ext.check_status("gemm_pair split-k accumulate")
    torch.testing.assert_close(acc, ref + 2.0, rtol=1e-3, atol=2e-2)


def test_device_barrier_gives_up_with_a_status_when_the_peer_never_signals():
    """Failure detection on the device: the barrier of rank 0 in a 2-rank table whose second signal pad nobody ever writes
    runs into its time limit, records status 5 (peer wait) and returns; the context stays usable and the host-side check
    turns the status into an exception."""
    from verl_b200.ops import _ext

    o = _ext.ops()
    _ext.check_status("before")
    my_pad = torch.zeros(1024, dtype=torch.int32, device="cuda")
    absent_peer_pad = torch.zeros(1024, dtype=torch.int32, device="cuda")
    table = torch.tensor([my_pad.data_ptr(), absent_peer_pad.data_ptr()], dtype=torch.int64)
    import time

    t0 = time.time()
    o.symm_barrier(table, 0, 2, 1)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.0 < waited < 10.0, waited                              # gave up after its ~2 s limit instead of spinning forever
    assert int(absent_peer_pad[0]) == 1 and int(my_pad[0]) == 1     # this rank did announce itself to both pads
    with pytest.raises(RuntimeError, match="status 5"):
        _ext.check_status("barrier without a peer")
    _ext.check_status("status word was cleared by the failed check")
    assert float(torch.ones(8, device="cuda").sum()) == 8.0         # the context is still usable
