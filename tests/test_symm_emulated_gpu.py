"""The multi-rank kernels on ONE GPU: the "peers" of every pointer table are separate buffers of the same device, and one
process plays each rank in turn. No launch here waits for a later launch: the kernels that only read or write peers are
order-free, and the signalled all-reduce is driven phase by phase (every rank's GEMM + signal first, every rank's slot sum
after), so all flags are already set when a waiter starts. What this covers is the addressing of every rank's view (offsets,
slot parity, epochs, head routing tables, K segments); the NVLink transport itself is covered by the tests that need two
devices."""

import pytest
import torch

pytestmark = pytest.mark.gpu

W = 2


@pytest.fixture(scope="module")
def o():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from verl_b200.ops import _ext

    _ext.load()
    return _ext.ops()


def _table(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64)


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


def _status_clean(o):
    torch.cuda.synchronize()
    assert int(o.take_status()) == 0


def test_reduce_scatter_scale_and_sumsq(o):
    torch.manual_seed(0)
    n = 1 << 20
    grads = [torch.randn(n, device="cuda") for _ in range(W)]
    want = sum(grads) / W
    for r in range(W):
        shard = torch.full((n // W + 8,), 7.0, device="cuda")          # 8 canary words behind the shard
        tot = torch.zeros(1, device="cuda")
        o.symm_reduce_scatter(_table(grads), W, r * (n // W), shard[: n // W], tot, 1.0 / W)
        ref = want[r * (n // W):(r + 1) * (n // W)]
        assert torch.allclose(shard[: n // W], ref, atol=1e-6)
        assert torch.all(shard[n // W:] == 7.0)
        assert abs(tot.item() - ref.double().pow(2).sum().item()) / ref.double().pow(2).sum().item() < 1e-5
    _status_clean(o)


def test_adamw_allgather_writes_every_ranks_parameter_copy(o):
    torch.manual_seed(1)
    n = 1 << 18
    sh = n // W
    params = [torch.zeros(n + 16, device="cuda", dtype=torch.bfloat16) for _ in range(W)]      # 16 canary elements at the end
    for p in params:
        p[n:] = 3.0
    p32 = torch.randn(n, device="cuda") * 0.02
    g = torch.randn(n, device="cuda") * 0.01
    m0, v0 = torch.randn(n, device="cuda") * 1e-3, torch.rand(n, device="cuda") * 1e-5
    scalars = torch.tensor([0.5, 0.0], device="cuda")                  # clip coefficient 0.5, no skip
    hp = dict(lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, wd=0.01, step=3)
    # oracle: the single-GPU AdamW kernel on the whole vector
    rp, rm, rv, r16 = p32.clone(), m0.clone(), v0.clone(), torch.empty(n, device="cuda", dtype=torch.bfloat16)
    o.adamw_(rp, rm, rv, g, r16, hp["lr"], hp["b1"], hp["b2"], hp["eps"], hp["wd"], hp["step"], scalars)
    for r in range(W):
        sl = slice(r * sh, (r + 1) * sh)
        lp, lm, lv = p32[sl].clone(), m0[sl].clone(), v0[sl].clone()
        o.symm_adamw_allgather(lp, lm, lv, g[sl].contiguous(), _table(params), W, r * sh, hp["lr"], hp["b1"], hp["b2"], hp["eps"], hp["wd"],
                               hp["step"], scalars)
        assert torch.allclose(lp, rp[sl], atol=1e-7) and torch.allclose(lm, rm[sl], atol=1e-8) and torch.allclose(lv, rv[sl], atol=1e-10)
    for p in params:
        assert (p[:n].float() - r16.float()).abs().max().item() < 2e-4 and torch.all(p[n:] == 3.0)
    assert torch.equal(params[0], params[1])
    # skip flag set (a non-finite gradient norm): state stays as it is, the parameter copies are rewritten with the same values
    before = [p.clone() for p in params]
    lp, lm, lv = rp[:sh].clone(), rm[:sh].clone(), rv[:sh].clone()
    o.symm_adamw_allgather(lp, lm, lv, g[:sh].contiguous(), _table(params), W, 0, 1e-3, 0.9, 0.95, 1e-8, 0.01, 4,
                           torch.tensor([1.0, 1.0], device="cuda"))
    assert torch.equal(lp, rp[:sh]) and torch.equal(lm, rm[:sh]) and torch.equal(lv, rv[:sh])
    assert all(torch.equal(a, b) for a, b in zip(params, before))
    _status_clean(o)


@pytest.mark.parametrize("staged", [False, True])
def test_allgather_a_and_b_fused_into_the_gemm(o, staged):
    torch.manual_seed(2)
    T, H, N = 512, 1024, 768
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, H, device="cuda")).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    ref = x.float() @ w.float().t()
    x_seg = [x[r * (T // W):(r + 1) * (T // W)].contiguous() for r in range(W)]
    w_seg = [w[r * (N // W):(r + 1) * (N // W)].contiguous() for r in range(W)]
    for r in range(W):
        stage_a = torch.empty(T * H, device="cuda", dtype=torch.bfloat16) if staged else None
        flags_a = torch.zeros(T // 128 + 8, device="cuda", dtype=torch.int32) if staged else None
        stage_b = torch.empty(N * H, device="cuda", dtype=torch.bfloat16) if staged else None
        flags_b = torch.zeros(N // 128 + 8, device="cuda", dtype=torch.int32) if staged else None
        stage_t = torch.empty(T * H, device="cuda", dtype=torch.bfloat16) if staged else None
        flags_t = torch.zeros(T // 128 + 8, device="cuda", dtype=torch.int32) if staged else None     # a flag counts the calls on its buffer
        for ep in (1, 2, 3):        # staging flags carry the epoch: later calls must not trust rows staged by earlier ones
            xs = [s * ep for s in x_seg]
            out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            o.gemm_allgather_a(_table(xs), T // W, w, out, bias, r, stage_a, flags_a, ep)
            assert _rel(out, ep * ref + bias.float()) < 1e-2, (r, ep)
            if staged:      # the same product from the weight stored [K, N] (backward of a row-parallel layer); the peers' rows
                outt = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)     # of the gathered operand are left in the staging buffer
                o.gemm_allgather_a(_table(xs), T // W, w.t().contiguous(), outt, None, r, stage_t, flags_t, ep, True)
                assert _rel(outt, ep * ref) < 1e-2, (r, ep)
                got = stage_t.view(T, H)
                for q in range(W):
                    if q != r:
                        assert torch.equal(got[q * (T // W):(q + 1) * (T // W)], xs[q])
            out2 = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            ws = [s * ep for s in w_seg]
            o.gemm_allgather_b(x, _table(ws), N // W, out2, None, r, stage_b, flags_b, ep)
            assert _rel(out2, ep * ref) < 1e-2, (r, ep)
    _status_clean(o)


@pytest.mark.parametrize("scatter_rows", [False, True])
def test_peer_scatter_epilogue_and_slot_sum(o, scatter_rows):
    """GEMM → all-reduce (every rank receives all rows) and GEMM → reduce-scatter (rank j receives row block j)."""
    torch.manual_seed(3)
    T, H, N = 256, 1024, 384
    Kl = H // W
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, H, device="cuda")).bfloat16()
    ref = x.float() @ w.float().t()
    rows = T // W if scatter_rows else T
    slot_elems = rows * N + 64                                        # slack between slots: must stay untouched
    slots = [torch.full((W * slot_elems,), 9.0, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    for r in range(W):                                                # rank r owns K slice r and writes slot r of every receiver
        xk, wk = x[:, r * Kl:(r + 1) * Kl].contiguous(), w[:, r * Kl:(r + 1) * Kl].contiguous()
        if r % 2 == 0:
            o.gemm_peer_scatter(xk, wk, _table(slots), r, T // W if scatter_rows else 0, slot_elems)
        else:               # odd ranks pass the weight slice stored [K, N] (the layout an activation-gradient GEMM sees)
            o.gemm_peer_scatter(xk, wk.t().contiguous(), _table(slots), r, T // W if scatter_rows else 0, slot_elems, True)
    res = torch.randn(rows, N, device="cuda").bfloat16()
    for r in range(W):
        out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
        o.slots_reduce(slots[r], W, slot_elems, rows, N, None if scatter_rows else res, out)
        want = ref[r * rows:(r + 1) * rows] if scatter_rows else ref + res.float()
        assert _rel(out, want) < 2e-2, r
        for s in range(W):
            assert torch.all(slots[r][s * slot_elems + rows * N:(s + 1) * slot_elems] == 9.0)
    _status_clean(o)


@pytest.mark.parametrize("T,split_k", [(256, 0), (64, 4)])
def test_signalled_allreduce_over_seven_epochs(o, T, split_k):
    """Slot parity, the epoch in the signal pad and the per-rank flags over back-to-back calls with different data."""
    torch.manual_seed(4)
    H, N = 4096, 512
    Kl = H // W
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, H, device="cuda")).bfloat16()
    ref = x.float() @ w.float().t()
    res = torch.randn(T, N, device="cuda").bfloat16()
    half = 4 * T * N
    slots = [torch.zeros(2 * half, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    sigs = [torch.zeros(64, device="cuda", dtype=torch.int32) for _ in range(W)]
    xs = [x[:, r * Kl:(r + 1) * Kl].contiguous() for r in range(W)]
    ws = [w[:, r * Kl:(r + 1) * Kl].contiguous() for r in range(W)]
    for i in range(7):
        outs = [torch.empty(T, N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
        for r in range(W):          # phase 1 on every rank: partial product into the own slot, signal into every pad
            o.gemm_allreduce_sig(xs[r] * (i + 1), ws[r], _table(slots), _table(sigs), r, half, slots[r], sigs[r], res, outs[r], 0, split_k, 4, 1)
        for r in range(W):          # phase 2 on every rank: all flags are set by now, the sum pulls the peers' partials
            o.gemm_allreduce_sig(xs[r], ws[r], _table(slots), _table(sigs), r, half, slots[r], sigs[r], res, outs[r], 0, split_k, 4, 2)
        for r in range(W):
            assert _rel(outs[r], (i + 1) * ref + res.float()) < 2e-2, (i, r)
    _status_clean(o)


def test_ulysses_head_scatter_and_k_segmented_gather(o):
    """QKV projection whose epilogue routes every head to its owner, and the output projection that reads its A operand
    from the ranks holding the head slices; together they are the two all-to-alls of sequence parallelism."""
    torch.manual_seed(5)
    D, Hq, Hkv, hidden = 128, 4, 2, 512
    hq_l, hkv_l = Hq // W, Hkv // W
    Cl, Kl = (hq_l + 2 * hkv_l) * D, hq_l * D
    Tl = 256
    Tp = Tl * W
    x = torch.randn(Tp, hidden, device="cuda").bfloat16()
    w_qkv = (0.05 * torch.randn((Hq + 2 * Hkv) * D, hidden, device="cuda")).bfloat16()
    b_qkv = torch.randn((Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    rank_of = [h // hq_l for h in range(Hq)] + [j // hkv_l for _ in range(2) for j in range(Hkv)]
    slot_of = [h % hq_l for h in range(Hq)] + [base + j % hkv_l for base in (hq_l, hq_l + hkv_l) for j in range(Hkv)]
    bufs = [torch.full((Tp * Cl + 64,), 5.0, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    for r in range(W):
        o.gemm_head_scatter(x[r * Tl:(r + 1) * Tl].contiguous(), w_qkv, b_qkv, _table(bufs), Cl, r * Tl, D,
                            torch.tensor(rank_of, dtype=torch.int32), torch.tensor(slot_of, dtype=torch.int32))
    full = (x.float() @ w_qkv.float().t() + b_qkv.float()).view(Tp, Hq + 2 * Hkv, D)
    for r in range(W):
        heads = [h for h in range(Hq + 2 * Hkv) if rank_of[h] == r]
        heads.sort(key=lambda h: slot_of[h])
        want = full[:, heads].reshape(Tp, Cl)
        assert _rel(bufs[r][: Tp * Cl].view(Tp, Cl), want) < 1e-2, r
        assert torch.all(bufs[r][Tp * Cl:] == 5.0)
    # output projection: rank r holds the attention output of its heads for ALL tokens
    o_all = torch.randn(Tp, Hq * D, device="cuda").bfloat16()
    w_o = (0.05 * torch.randn(hidden, Hq * D, device="cuda")).bfloat16()
    o_bufs = [o_all[:, r * Kl:(r + 1) * Kl].contiguous() for r in range(W)]
    ref = o_all.float() @ w_o.float().t()
    for r in range(W):
        stage = torch.empty((Tl + 128) * Hq * D, device="cuda", dtype=torch.bfloat16)
        flags = torch.zeros(((Tl + 128) // 128) * W + 8, device="cuda", dtype=torch.int32)
        for ep, st in ((1, None), (1, stage), (2, stage)):
            out = torch.empty(Tl, hidden, device="cuda", dtype=torch.bfloat16)
            o.gemm_kseg(_table(o_bufs), Kl, Tp, r * Tl, w_o, out, None, r, st, flags if st is not None else None, ep)
            assert _rel(out, ref[r * Tl:(r + 1) * Tl]) < 1e-2, (r, ep)
        out = torch.empty(Tl, hidden, device="cuda", dtype=torch.bfloat16)
        o.gemm_kseg(_table(o_bufs), Kl, Tp, r * Tl, w_o.t().contiguous(), out, None, r, stage, flags, 3, True)      # weight stored [K, N]
        assert _rel(out, ref[r * Tl:(r + 1) * Tl]) < 1e-2, r
    # backward of the output projection: (dY @ W_o) with the sequence -> head routing in the epilogue, W_o as the forward stores it
    dy = torch.randn(Tp, hidden, device="cuda").bfloat16()
    dbufs = [torch.full((Tp * Kl + 64,), 5.0, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    q_rank = torch.tensor([h // hq_l for h in range(Hq)], dtype=torch.int32)
    q_slot = torch.tensor([h % hq_l for h in range(Hq)], dtype=torch.int32)
    for r in range(W):
        o.gemm_head_scatter(dy[r * Tl:(r + 1) * Tl].contiguous(), w_o, None, _table(dbufs), Kl, r * Tl, D, q_rank, q_slot, True)
    want = dy.float() @ w_o.float()
    for r in range(W):
        assert _rel(dbufs[r][: Tp * Kl].view(Tp, Kl), want[:, r * Kl:(r + 1) * Kl]) < 1e-2, r
        assert torch.all(dbufs[r][Tp * Kl:] == 5.0)
    _status_clean(o)


@pytest.mark.parametrize("T0,T1", [(300, 300), (257, 90)])
def test_moe_dispatch_and_combine_fused_into_the_grouped_gemms(o, T0, T1):
    """Expert parallelism over two emulated ranks: the gate/up grouped GEMM fetches its rows from the "ranks" that hold the tokens,
    the down-projection's epilogue stores weighted rows into the owners' slot buffers; the slot sums must equal a dense fp32
    evaluation of the same routing. The transposed-weight variants (the two GEMMs of the backward pass) are checked the same way."""
    from verl_b200.ops.moe import ep_row_tables

    torch.manual_seed(6)
    H, I, E, k = 512, 256, 8, 2
    e_local = E // W
    Ts = [T0, T1]
    Tc = max(Ts)
    xs = [torch.randn(Tc, H, device="cuda").bfloat16() for _ in range(W)]            # token buffers (rows >= T are never addressed)
    gate_up = (0.05 * torch.randn(E, 2 * I, H, device="cuda")).bfloat16()
    down = (0.05 * torch.randn(E, H, I, device="cuda")).bfloat16()
    idx_all = torch.full((W, Tc, k), -1, dtype=torch.long, device="cuda")
    w_all = torch.zeros(W, Tc, k, device="cuda")
    for r in range(W):
        idx_all[r, : Ts[r]] = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(Ts[r])])
        w_all[r, : Ts[r]] = torch.rand(Ts[r], k, device="cuda") + 0.1
    cbufs = [torch.full((k * Tc * H + 64,), 7.0, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    gbufs = [torch.full((k * Tc * H + 64,), 7.0, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    acts = []
    for r in range(W):
        row_src, row_dst, row_w, blk, rng = ep_row_tables(idx_all, w_all, r, e_local)
        R = row_src.numel()
        stage = torch.empty(R, H, device="cuda", dtype=torch.bfloat16)
        flags = torch.empty(R // 128, device="cuda", dtype=torch.int32)
        gu_l, dn_l = gate_up[r * e_local:(r + 1) * e_local].contiguous(), down[r * e_local:(r + 1) * e_local].contiguous()
        h = o.gemm_grouped_dispatch(_table(xs), H, row_src, gu_l, blk, stage, flags, False)
        # the staged operand is the gathered token rows (zeros on padding rows)
        used = row_src >= 0
        src_rank, src_tok = (row_src[used] >> 24).long(), (row_src[used] & 0xFFFFFF).long()
        want_rows = torch.stack(xs)[src_rank, src_tok]
        blk_used = (blk >= 0).repeat_interleave(128)
        assert torch.equal(stage[used], want_rows) and torch.all(stage[blk_used & ~used] == 0)
        e_of_row = blk.long().repeat_interleave(128)[used]
        want_h = torch.einsum("rh,rnh->rn", want_rows.float(), gu_l.float()[e_of_row])
        assert _rel(h[used], want_h) < 1e-2
        a = o.swiglu_fwd(h)
        o.gemm_grouped_combine(a, dn_l, blk, row_dst, row_w, _table(cbufs), H, False)
        acts.append((a, row_src, row_dst, row_w, blk, used, e_of_row, dn_l, gu_l, h))
        # backward-direction variants: input gradients through the transposed weights
        da = o.gemm_grouped_dispatch(_table(xs), H, row_src, dn_l, blk, stage, flags, True)             # [R, I] = rows @ down[e]
        want_da = torch.einsum("rh,rhi->ri", want_rows.float(), dn_l.float()[e_of_row])
        assert _rel(da[used], want_da) < 1e-2
        ones = (row_dst >= 0).float()
        o.gemm_grouped_combine(h, gu_l, blk, row_dst, ones, _table(gbufs), H, True)                      # rows of h @ gate_up[e] -> owners
    torch.cuda.synchronize()
    for r in range(W):
        T = Ts[r]
        y = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
        o.slots_reduce(cbufs[r][: k * Tc * H], k, Tc * H, T, H, None, y)
        x = xs[r][:T].float()
        want = torch.zeros(T, H, device="cuda")
        want_g = torch.zeros(T, H, device="cuda")
        for j in range(k):
            e = idx_all[r, :T, j]
            hh = torch.einsum("th,tnh->tn", x, gate_up.float()[e])
            hb = hh.bfloat16().float()
            act = (torch.nn.functional.silu(hb[:, :I]) * hb[:, I:]).bfloat16().float()
            want += w_all[r, :T, j, None] * torch.einsum("ti,thi->th", act, down.float()[e])
            want_g += torch.einsum("tn,tnh->th", hb, gate_up.float()[e])
        assert _rel(y, want) < 2e-2, r
        g = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
        o.slots_reduce(gbufs[r][: k * Tc * H], k, Tc * H, T, H, None, g)
        assert _rel(g, want_g) < 2e-2, r
        assert torch.all(cbufs[r][k * Tc * H:] == 7.0) and torch.all(gbufs[r][k * Tc * H:] == 7.0)
    _status_clean(o)
