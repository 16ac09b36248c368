"""Micro-benchmarks of the sm_100a kernels: CUDA-event timing after warm-up with an L2 flush between iterations,
reported as achieved TFLOP/s or GB/s and as a fraction of the measured machine peaks (``MEASURED_PEAKS.json`` at the
repository root: cuBLAS bf16 burst throughput and STREAM-style copy bandwidth; fallbacks 1590 TFLOP/s and 6650 GB/s).

    python -m verl_b200.ops.kernel_bench gemm --m 8192 --n 8192 --k 4096
    python -m verl_b200.ops.kernel_bench all

The same entry point is what the committed ``profiles/*.md`` summaries were captured with (under ``ncu``, one kernel,
small case).
"""

from __future__ import annotations

import argparse
import json
import math
import os

import torch


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "of measured"
    return 1590.0, 6650.0, "of fallback"


def timeit(fn, iters=10, warmup=3, flush=True):
    buf = torch.empty(64 * 1024 * 1024, device="cuda", dtype=torch.float32) if flush else None   # 256 MB > L2
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            buf.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def report(name, ms, flops=None, bytes_=None):
    tf, gbs, tag = peaks()
    msg = f"{name}: {ms * 1e3:.1f} us"
    if flops:
        a = flops / ms / 1e9
        msg += f"  {a:.0f} TFLOP/s ({a / tf:.2f} {tag} cuBLAS bf16)"
    if bytes_:
        a = bytes_ / ms / 1e6
        msg += f"  {a:.0f} GB/s ({a / gbs:.2f} {tag} copy bandwidth)"
    print(msg, flush=True)


def bench_gemm(a):
    from verl_b200.ops import _ext

    o = _ext.ops()
    M, N, K = a.m, a.n, a.k
    x = (torch.randn(K, M, device="cuda") if a.a_mn else torch.randn(M, K, device="cuda")).bfloat16()
    w = (torch.randn(K, N, device="cuda") if a.b_mn else torch.randn(N, K, device="cuda")).bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.float32 if a.f32 else torch.bfloat16)
    ms = timeit(lambda: o.gemm(x, w, out, None, a.a_mn, a.b_mn, False, a.bn), a.iters)
    report(f"gemm M={M} N={N} K={K} a_mn={a.a_mn} b_mn={a.b_mn}", ms, flops=2.0 * M * N * K)
    if a.compare:
        A = x.t() if a.a_mn else x
        B = w if a.b_mn else w.t()
        ms2 = timeit(lambda: torch.matmul(A, B), a.iters)
        report("  cuBLAS (torch.matmul) same shape", ms2, flops=2.0 * M * N * K)


class _SmiSampler:
    """SM clock and board power read through NVML (read-only queries) every 20 ms while a sustained loop runs."""

    def __init__(self):
        import threading

        self.samples, self._stop, self._th = [], threading.Event(), None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv, self._h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        except Exception:  # noqa: BLE001
            self._nv = None
        if self._nv is not None:
            self._th = threading.Thread(target=self._run, daemon=True)
            self._th.start()

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append((nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0))
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(0.02)

    def stop(self):
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=1)
        tail = self.samples[len(self.samples) // 2:]           # second half: the steady state
        if not tail:
            return None, None
        mhz = sorted(x[0] for x in tail)[len(tail) // 2]
        watts = sorted(x[1] for x in tail)[len(tail) // 2]
        return mhz, watts


LAST_SUSTAINED = {"sm_mhz": None, "watts": None}


def sustained(fn, seconds=1.5):
    """Back-to-back launches for about ``seconds`` (no flush, operands larger than L2): the power-capped steady state a
    kernel sees inside a long training step. Returns milliseconds per launch; the median SM clock and board power of the
    second half of the loop are left in ``LAST_SUSTAINED``."""
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    n = max(8, int(seconds * 1e3 / max(s.elapsed_time(e), 1e-3)))
    smp = _SmiSampler()
    s.record()
    for _ in range(n):
        fn()
    e.record()
    torch.cuda.synchronize()
    LAST_SUSTAINED["sm_mhz"], LAST_SUSTAINED["watts"] = smp.stop()
    return s.elapsed_time(e) / n


def bench_gemm_layer(a):
    """The GEMMs of one decoder layer (hidden --k, FFN --ffn, q/kv heads) on --m tokens in their three roles: forward
    (x W^T), input gradient (dy W) and weight gradient (dy^T x accumulated into fp32), own kernel vs torch.matmul, as a burst
    (median of flushed single launches) and sustained (back-to-back for 1.5 s)."""
    from verl_b200.ops import _ext

    o = _ext.ops()
    T, H, I = a.m, a.k, a.ffn
    D = 128
    shapes = [("qkv", (a.heads + 2 * a.kv_heads) * D, H), ("o", H, a.heads * D), ("gate_up", 2 * I, H), ("down", H, I)]
    tot = {"own": 0.0, "lib": 0.0}
    print(f"| projection | role | M x N x K | own burst us | cuBLAS burst us | own sustained us | cuBLAS sustained us | own/cuBLAS sustained |")
    print("|---|---|---|---|---|---|---|---|")
    for name, N, K in shapes:
        x = torch.randn(T, K, device="cuda").bfloat16()
        w = (0.02 * torch.randn(N, K, device="cuda")).bfloat16()
        dy = torch.randn(T, N, device="cuda").bfloat16()
        y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
        dw = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        roles = [
            ("fwd", (T, N, K), lambda: o.gemm(x, w, y, None, False, False, False, a.bn), lambda: torch.matmul(x, w.t(), out=y)),
            ("dgrad", (T, K, N), lambda: o.gemm(dy, w, dx, None, False, True, False, a.bn), lambda: torch.matmul(dy, w, out=dx)),
            ("wgrad", (N, K, T), lambda: o.gemm(dy, x, dw, None, True, True, True, a.bn), lambda: torch.matmul(dy.t(), x)),
        ]
        for role, (m, n, k), own, lib in roles:
            fl = 2.0 * m * n * k
            b_own, b_lib = timeit(own, a.iters), timeit(lib, a.iters)
            s_own = sustained(own)
            c_own = dict(LAST_SUSTAINED)
            s_lib = sustained(lib)
            c_lib = dict(LAST_SUSTAINED)
            tot["own"] += s_own
            tot["lib"] += s_lib
            print(f"| {name} | {role} | {m}x{n}x{k} | {b_own * 1e3:.1f} ({fl / b_own / 1e9:.0f} TF) | {b_lib * 1e3:.1f} ({fl / b_lib / 1e9:.0f} TF) | "
                  f"{s_own * 1e3:.1f} ({fl / s_own / 1e9:.0f} TF, {c_own['sm_mhz']} MHz, {c_own['watts'] or 0:.0f} W) | "
                  f"{s_lib * 1e3:.1f} ({fl / s_lib / 1e9:.0f} TF, {c_lib['sm_mhz']} MHz, {c_lib['watts'] or 0:.0f} W) | {s_lib / s_own:.2f} |", flush=True)
    print(f"layer total sustained: own {tot['own'] * 1e3:.0f} us, cuBLAS {tot['lib'] * 1e3:.0f} us, ratio {tot['lib'] / tot['own']:.3f} "
          "(the cuBLAS weight-gradient column is a bf16-output matmul without the fp32 accumulation the own kernel fuses)")


def bench_layer_step(a):
    """Forward + backward of ONE decoder layer of the --model preset on --m packed tokens (sequences of --seqlen), weight
    gradients accumulated into fp32 ``main_grad`` buffers exactly as the training engine does. This is the unit whose
    launch list (``ncu --metrics gpu__time_duration.sum``) shows each kernel's share of a training step."""
    from verl_b200.models.config import PRESETS
    from verl_b200.models.transformer import DecoderLayer, PackedBatch
    from verl_b200 import ops

    cfg = PRESETS[a.model]
    layer = DecoderLayer(cfg, torch.bfloat16, "cuda", 0)
    with torch.no_grad():
        for n_, p_ in layer.named_parameters():
            if n_.endswith("layernorm"):
                p_.fill_(1.0)
            elif n_.endswith("bias"):
                p_.zero_()
            else:
                p_.normal_(0.0, 0.02)
    for p_ in layer.parameters():
        p_.main_grad = torch.zeros(p_.shape, device="cuda", dtype=torch.float32)
    T, L = a.m, a.seqlen
    lens = [L] * (T // L) + ([T % L] if T % L else [])
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    pos = torch.cat([torch.arange(n_, dtype=torch.int32) for n_ in lens]).cuda()
    pb = PackedBatch(torch.zeros(T, dtype=torch.long, device="cuda"), pos, cu.cuda(), cu, max(lens))
    cos, sin = ops.rope_tables(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta, "cuda")
    h0 = torch.randn(T, cfg.hidden_size, device="cuda").bfloat16()
    r0 = torch.randn(T, cfg.hidden_size, device="cuda").bfloat16()
    g = torch.randn(T, cfg.hidden_size, device="cuda").bfloat16()

    def fwd():
        with torch.no_grad():
            layer(h0, r0, pb, cos, sin)

    def fwdbwd():
        h = h0.clone().requires_grad_(True)
        r = r0.clone().requires_grad_(True)
        m, res = layer(h, r, pb, cos, sin)
        torch.autograd.backward([m, res], [g, g])

    n_par = sum(p_.numel() for n_, p_ in layer.named_parameters() if p_.dim() == 2)
    attn = sum(2 * 2 * l * l / 2 * cfg.head_dim * cfg.num_attention_heads for l in lens)
    ms_f = sustained(fwd, 1.0) if a.sustained else timeit(fwd, a.iters)
    report(f"decoder layer fwd {a.model} T={T} (GEMM + causal attention FLOPs)", ms_f, flops=2.0 * n_par * T + attn)
    ms_b = sustained(fwdbwd, 1.0) if a.sustained else timeit(fwdbwd, a.iters)
    report(f"decoder layer fwd+bwd {a.model} T={T}", ms_b, flops=6.0 * n_par * T + 3.5 * attn)


def bench_gemm_fp8(a):
    """e4m3 GEMM (per-row / per-column scales in the epilogue) against the bf16 kernel and torch._scaled_mm on the same shape."""
    from verl_b200.ops import _ext
    from verl_b200.ops.quant import rowwise_cast_to_fp8

    o = _ext.ops()
    M, N, K = a.m, a.n, a.k
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    a8, sa = rowwise_cast_to_fp8(x)
    b8, sb = rowwise_cast_to_fp8(w)
    ms = timeit(lambda: o.gemm_fp8(a8, b8, sa, sb, None, False), a.iters)
    report(f"gemm fp8 e4m3 M={M} N={N} K={K} (row/col scales, bf16 out)", ms, flops=2.0 * M * N * K)
    ms_c = timeit(lambda: o.fp8_row_cast(x), a.iters)
    report(f"  per-token e4m3 cast [{M}x{K}]", ms_c, bytes_=M * K * 3.0)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms_b = timeit(lambda: o.gemm(x, w, out, None, False, False, False, 0), a.iters)
    report("  bf16 kernel, same shape", ms_b, flops=2.0 * M * N * K)
    from verl_b200.ops.quant import act_cast_to_fp8, blockwise_cast_to_fp8

    a8b, sab = act_cast_to_fp8(x)
    b8b, sbb = blockwise_cast_to_fp8(w)
    ms_blk = timeit(lambda: o.gemm_fp8_block(a8b, sab, b8b, sbb, None, False), a.iters)
    report("  block-scaled variant (1x128 activation / 128x128 weight scales, promotion per K block)", ms_blk, flops=2.0 * M * N * K)
    if a.compare:
        try:
            ms2 = timeit(lambda: torch._scaled_mm(a8, b8.t(), scale_a=sa[:, None], scale_b=sb[None, :], out_dtype=torch.bfloat16), a.iters)
            report("  cuBLASLt (torch._scaled_mm, row-wise scales) same shape", ms2, flops=2.0 * M * N * K)
        except Exception as e:  # noqa: BLE001
            print(f"  torch._scaled_mm unavailable: {type(e).__name__}: {str(e)[:120]}", flush=True)


def bench_attn(a, backward=False):
    from verl_b200 import ops

    Hq, Hkv, D = a.heads, a.kv_heads, 128
    lens = [a.seqlen] * a.batch
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    cud = cu.cuda()
    qkv = (0.5 * torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda")).bfloat16().requires_grad_(backward)
    fl = sum(2 * 2 * L * L / 2 * D * Hq for L in lens)
    if not backward:
        with torch.no_grad():
            ms = timeit(lambda: ops.attention_varlen(qkv, cud, Hq, Hkv, D, a.seqlen, cu), a.iters)
        report(f"attention fwd T={T} L={a.seqlen} {Hq}/{Hkv} heads (causal FLOPs)", ms, flops=fl)
    else:
        out = ops.attention_varlen(qkv, cud, Hq, Hkv, D, a.seqlen, cu)
        dout = torch.randn_like(out)
        ms = timeit(lambda: torch.autograd.grad(out, qkv, dout, retain_graph=True), a.iters)
        report(f"attention bwd T={T} L={a.seqlen} {Hq}/{Hkv} heads (causal FLOPs x2.5)", ms, flops=2.5 * fl)
    if a.compare:
        # the library kernel the reference calls for the same op (verl/models/transformers/monkey_patch.py:146-148)
        try:
            from flash_attn import flash_attn_varlen_func
        except ImportError as e:
            print(f"  flash_attn not importable: {e}")
            return
        q, k, v = (t.reshape(T, -1, D).contiguous() for t in qkv.detach().split([Hq * D, Hkv * D, Hkv * D], dim=-1))
        if not backward:
            with torch.no_grad():
                ms2 = timeit(lambda: flash_attn_varlen_func(q, k, v, cud, cud, a.seqlen, a.seqlen, causal=True), a.iters)
            report("  flash_attn_varlen_func fwd, same shapes", ms2, flops=fl)
        else:
            q, k, v = (t.requires_grad_(True) for t in (q, k, v))
            o2 = flash_attn_varlen_func(q, k, v, cud, cud, a.seqlen, a.seqlen, causal=True)
            d2 = torch.randn_like(o2)
            ms2 = timeit(lambda: torch.autograd.grad(o2, (q, k, v), d2, retain_graph=True), a.iters)
            report("  flash_attn_varlen_func bwd, same shapes", ms2, flops=2.5 * fl)


def bench_lmhead(a):
    from verl_b200 import ops

    M, V, K = a.m, a.vocab, a.k
    h = (0.5 * torch.randn(M, K, device="cuda")).bfloat16()
    w = (0.02 * torch.randn(V, K, device="cuda")).bfloat16()
    lab = torch.randint(0, V, (M,), device="cuda")
    with torch.no_grad():
        ms = timeit(lambda: ops.linear_logprob_entropy(h, w, lab, 1.0, True), a.iters)
    report(f"lm_head->logprob+entropy fwd M={M} V={V} K={K}", ms, flops=2.0 * M * V * K)
    if a.compare:
        # forward + backward of the whole op against two library formulations of the same thing
        hg = h.clone().requires_grad_(True)

        def own():
            lp, ent = ops.linear_logprob_entropy(hg, w, lab, 1.0, False)
            torch.autograd.grad(lp.sum(), hg)

        ms_o = timeit(own, a.iters)
        report("  own kernels fwd + bwd (d hidden; the weight gradient is a separate accumulate GEMM)", ms_o, flops=4.0 * M * V * K)

        def torch_ce():
            logits = torch.nn.functional.linear(hg, w).float()
            torch.autograd.grad(torch.nn.functional.cross_entropy(logits, lab, reduction="sum"), hg)

        if M * V * 6 < 40e9:
            report("  cuBLAS logits + torch cross_entropy fwd + bwd", timeit(torch_ce, a.iters), flops=4.0 * M * V * K)
        try:
            from liger_kernel.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Liger
        except ImportError as e:
            print(f"  liger_kernel not importable: {e}")
            return
        wg = w.clone().requires_grad_(True)

        def liger():
            out = Liger.apply(hg, wg, lab, None, None, -100, 0.0, 0.0, "sum")
            loss = out[0] if isinstance(out, tuple) else out
            torch.autograd.grad(loss, (hg, wg))

        report("  Liger fused linear + cross-entropy fwd + bwd (Triton; d hidden and d weight)", timeit(liger, a.iters), flops=6.0 * M * V * K)


def bench_decode_attn(a):
    from verl_b200.ops.attention import paged_decode_attention

    Hq, Hkv, D, B = a.heads, a.kv_heads, 128, a.batch
    blocks_per = (a.seqlen + 63) // 64 + 1
    nb = B * blocks_per + 1
    cache = torch.zeros(nb, 2, Hkv, 64, D, device="cuda", dtype=torch.bfloat16).normal_()
    bt = (torch.arange(B * blocks_per, device="cuda", dtype=torch.int32) + 1).reshape(B, blocks_per)
    kl = torch.full((B,), a.seqlen, dtype=torch.int32, device="cuda")
    q = torch.randn(B, Hq * D, device="cuda").bfloat16()
    out = torch.empty_like(q)
    ws = torch.empty(B * Hq * max(1, a.splits) * 130, device="cuda")
    ms = timeit(lambda: paged_decode_attention(q, cache, bt, kl, 1 / math.sqrt(D), a.splits, a.seqlen, ws, out, a.impl), a.iters)
    report(f"paged decode attention B={B} kv={a.seqlen} {Hq}/{Hkv} heads impl={a.impl}", ms, bytes_=B * a.seqlen * Hkv * D * 2 * 2)


def bench_elementwise(a):
    from verl_b200.ops import _ext, functional as Fn

    o = _ext.ops()
    T, H = a.m, a.k
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    report(f"rmsnorm fwd T={T} H={H}", timeit(lambda: Fn.rmsnorm(x, w, 1e-6), a.iters), bytes_=2 * T * H * 2)
    gu = torch.randn(T, 2 * H, device="cuda").bfloat16()
    report(f"swiglu fwd T={T} I={H}", timeit(lambda: Fn.swiglu(gu), a.iters), bytes_=3 * T * H * 2)
    n = T * H
    p32, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    sc = torch.tensor([1.0, 0.0, 0.0, 0.0], device="cuda")
    report(f"adamw n={n}", timeit(lambda: o.adamw_(p32, m, v, g, p16, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, sc), a.iters), bytes_=n * (4 * 4 + 3 * 4 + 2))


def bench_fused_gather(a):
    """Gather-fused GEMMs on ONE GPU: the "peers" are separate buffers in this GPU's memory, so the kernels run their full
    multi-rank code path (per-rank tensor maps, staging copies by the copy warps, arrival flags, head routing) without a
    second process. Used for single-GPU profiler captures of the fused kernels; NVLink figures come from
    ``verl_b200.parallel.comm_bench`` on real multi-GPU runs."""
    from verl_b200.ops import _ext

    o = _ext.ops()
    W, T, H, N = a.world, a.m, a.k, a.n
    Tl = T // W
    segs = [(torch.randn(Tl, H, device="cuda")).bfloat16() for _ in range(W)]
    ptrs = torch.tensor([s.data_ptr() for s in segs], dtype=torch.int64)
    w = (0.02 * torch.randn(N, H, device="cuda")).bfloat16()
    out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    stage = torch.empty(T * H, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(T // 128 + 8, device="cuda", dtype=torch.int32)
    ep = [0]

    def ag():
        ep[0] += 1
        o.gemm_allgather_a(ptrs, Tl, w, out, None, 0, stage, flags, ep[0])

    report(f"all-gather -> GEMM (staged, {W} segments on one GPU) M={T} N={N} K={H}", timeit(ag, a.iters), flops=2.0 * T * N * H)
    ref = torch.cat(segs).float() @ w.float().t()
    err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
    print(f"  max rel err vs fp32 matmul: {err:.2e}")
    # sequence -> head all-to-all fused into the QKV projection: every "rank" buffer is local
    D, Hq, Hkv = 128, a.heads, a.kv_heads
    C = (Hq + 2 * Hkv) * D
    wq = (0.02 * torch.randn(C, H, device="cuda")).bfloat16()
    hq_l, hkv_l = Hq // W, Hkv // W
    Cl = (hq_l + 2 * hkv_l) * D
    bufs = [torch.empty(T, Cl, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    optr = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64)
    rank_of = [h // hq_l for h in range(Hq)] + [j // hkv_l for j in range(Hkv)] * 2
    slot_of = [h % hq_l for h in range(Hq)] + [hq_l + j % hkv_l for j in range(Hkv)] + [hq_l + hkv_l + j % hkv_l for j in range(Hkv)]
    hr, hs = torch.tensor(rank_of, dtype=torch.int32), torch.tensor(slot_of, dtype=torch.int32)
    x = segs[0]
    report(f"QKV projection + head scatter ({W} destinations on one GPU) M={Tl} N={C} K={H}",
           timeit(lambda: o.gemm_head_scatter(x, wq, None, optr, Cl, 0, D, hr, hs), a.iters), flops=2.0 * Tl * C * H)


def bench_fused_emulated(a):
    """The other multi-rank kernels on ONE GPU at training sizes, every "peer" being a buffer of this GPU: gradient
    reduce-scatter (+ scale + squared norm), AdamW fused with the parameter all-gather, the peer-scatter GEMM epilogue with its
    slot sum (GEMM -> reduce-scatter), the signalled GEMM -> all-reduce pair at decode size, and the reshard + fp8 requantise
    kernel of the weight sync. The memory-bound ones are reported against the measured copy bandwidth with their algorithmic
    bytes; transport over NVLink is measured by ``verl_b200.parallel.comm_bench`` on real multi-GPU runs."""
    from verl_b200.ops import _ext

    o = _ext.ops()
    W = a.world
    tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64)      # noqa: E731
    # ---- gradient reduce-scatter: every rank reads its 1/W slice of all W gradient buffers (fp32) and writes it once
    n = 1 << 28                                                                         # 268M gradients = 1 GiB per "rank"
    grads = [torch.randn(n, device="cuda") for _ in range(W)]
    shard = torch.empty(n // W, device="cuda")
    tot = torch.zeros(1, device="cuda")
    ms = timeit(lambda: o.symm_reduce_scatter(tab(grads), W, 0, shard, tot, 1.0 / W), a.iters)
    report(f"symm_reduce_scatter {W} x {n // W} fp32 (reads {W} slices, writes one)", ms, bytes_=(W + 1) * (n // W) * 4.0)
    del grads
    # ---- AdamW + all-gather: p32/m/v read+write, g read, bf16 result written to all W parameter buffers
    sh = n // W
    p32, m, v, g = (torch.randn(sh, device="cuda") * 0.02 for _ in range(4))
    v = v.abs()
    params = [torch.empty(n, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    scal = torch.tensor([1.0, 0.0], device="cuda")
    ms = timeit(lambda: o.symm_adamw_allgather(p32, m, v, g, tab(params), W, 0, 1e-6, 0.9, 0.999, 1e-8, 0.01, 2, scal), a.iters)
    report(f"symm_adamw_allgather shard {sh} (3 fp32 r+w, 1 fp32 r, {W} bf16 w)", ms, bytes_=sh * (7 * 4.0 + W * 2.0))
    del p32, m, v, g, params, shard
    # ---- GEMM -> reduce-scatter: down projection of Qwen2.5-7B under TP = W (K split), rows scattered to their owners
    T, N, K = a.m, a.n, a.k // W
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (0.02 * torch.randn(N, K, device="cuda")).bfloat16()
    rows = T // W
    slot = rows * N
    slots = [torch.empty(W * slot, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    ms = timeit(lambda: o.gemm_peer_scatter(x, w, tab(slots), 0, rows, slot), a.iters)
    report(f"GEMM with peer-scatter epilogue (reduce-scatter form) M={T} N={N} K={K}", ms, flops=2.0 * T * N * K)
    out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: o.slots_reduce(slots[0], W, slot, rows, N, None, out), a.iters)
    report(f"slots_reduce {W} x [{rows}, {N}] bf16", ms, bytes_=(W + 1) * rows * N * 2.0)
    del slots
    # ---- decode-size GEMM -> all-reduce, signalled form, both emulated ranks per iteration
    Td = 256
    xd = torch.randn(Td, K, device="cuda").bfloat16()
    half = 8 * Td * N
    sl2 = [torch.zeros(2 * half, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    sig = [torch.zeros(64, device="cuda", dtype=torch.int32) for _ in range(W)]
    outs = [torch.empty(Td, N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]

    def ar():
        for r in range(W):
            o.gemm_allreduce_sig(xd, w, tab(sl2), tab(sig), r, half, sl2[r], sig[r], None, outs[r], 0, 0, 8, 1)
        for r in range(W):
            o.gemm_allreduce_sig(xd, w, tab(sl2), tab(sig), r, half, sl2[r], sig[r], None, outs[r], 0, 0, 8, 2)

    ms = timeit(ar, a.iters)
    report(f"signalled GEMM -> all-reduce, {W} emulated ranks back to back (2 x {W} launches) M={Td} N={N} K={K}", ms,
           bytes_=W * (N * K * 2.0 + Td * K * 2.0))
    # ---- weight sync: gather rows from W row shards + 128 x 128 block-fp8 requantise (gate_up of Qwen2.5-7B)
    Nw, Kw = 37888, 3584
    shards = [(0.02 * torch.randn(Nw // W, Kw, device="cuda")).bfloat16() for _ in range(W)]
    like = shards[0]
    ms = timeit(lambda: o.reshard_quant(tab(shards), Nw // W, Kw, 0, Nw, Kw, True, False, like), a.iters)
    report(f"reshard_quant {W} shards -> [{Nw}, {Kw}] e4m3 + block scales", ms, bytes_=Nw * Kw * 3.0)
    ms = timeit(lambda: o.reshard_quant(tab(shards), Nw // W, Kw, 0, Nw, Kw, False, True, like), a.iters)
    report(f"reshard (bf16 copy) {W} shards -> [{Nw}, {Kw}]", ms, bytes_=Nw * Kw * 4.0)
    torch.cuda.synchronize()
    _ext.check_status("fused_emulated")


def bench_fused_routed(a):
    """The routed variants of the fused GEMMs on ONE GPU, every "peer" being a buffer of this GPU: QKV projection with the
    sequence -> head routing in its epilogue, output projection reading its K-segmented operand from the head owners, and the two
    grouped GEMMs of an expert-parallel MoE layer (row gather from the token owners into the gate/up GEMM, weighted row scatter
    from the down projection). Qwen2.5-7B attention shapes / Qwen3-30B-A3B expert shapes; NVLink transport is measured by
    ``verl_b200.parallel.comm_bench``."""
    from verl_b200.ops import _ext
    from verl_b200.ops.moe import ep_row_tables

    o = _ext.ops()
    W = a.world
    tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64)      # noqa: E731
    D, Hq, Hkv, H = 128, 28, 4, 3584
    hq_l, hkv_l = Hq // W, Hkv // W
    Cl, Kl = (hq_l + 2 * hkv_l) * D, hq_l * D
    Tl = a.m // W
    Tp = Tl * W
    x = torch.randn(Tl, H, device="cuda").bfloat16()
    w_qkv = (0.02 * torch.randn((Hq + 2 * Hkv) * D, H, device="cuda")).bfloat16()
    rank_of = [h // hq_l for h in range(Hq)] + [j // hkv_l for _ in range(2) for j in range(Hkv)]
    slot_of = [h % hq_l for h in range(Hq)] + [base + j % hkv_l for base in (hq_l, hq_l + hkv_l) for j in range(Hkv)]
    hr, hs = torch.tensor(rank_of, dtype=torch.int32), torch.tensor(slot_of, dtype=torch.int32)
    bufs = [torch.empty(Tp * Cl, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    ms = timeit(lambda: o.gemm_head_scatter(x, w_qkv, None, tab(bufs), Cl, 0, D, hr, hs), a.iters)
    report(f"QKV projection with head-scatter epilogue M={Tl} N={(Hq + 2 * Hkv) * D} K={H}", ms, flops=2.0 * Tl * H * (Hq + 2 * Hkv) * D)
    o_bufs = [torch.randn(Tp, Kl, device="cuda").bfloat16() for _ in range(W)]
    w_o = (0.02 * torch.randn(H, Hq * D, device="cuda")).bfloat16()
    Tl_pad = (Tl + 127) // 128 * 128
    stage = torch.empty(Tl_pad * Hq * D, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros((Tl_pad // 128) * W + 8, device="cuda", dtype=torch.int32)
    out = torch.empty(Tl, H, device="cuda", dtype=torch.bfloat16)
    ep = [0]

    def kseg():
        ep[0] += 1
        o.gemm_kseg(tab(o_bufs), Kl, Tp, 0, w_o, out, None, 0, stage, flags, ep[0])

    ms = timeit(kseg, a.iters)
    report(f"output projection with K-segmented staged gather M={Tl} N={H} K={Hq * D}", ms, flops=2.0 * Tl * H * Hq * D)
    del bufs, o_bufs, stage
    # ---- expert-parallel MoE layer: 128 experts, top-8, hidden 2048, expert FFN 768
    Hm, I, E, k = 2048, 768, 128, 8
    e_local = E // W
    T = a.m
    xs = [torch.randn(T, Hm, device="cuda").bfloat16() for _ in range(W)]
    gate_up = (0.02 * torch.randn(e_local, 2 * I, Hm, device="cuda")).bfloat16()
    down = (0.02 * torch.randn(e_local, Hm, I, device="cuda")).bfloat16()
    idx_all = torch.stack([torch.rand(T, E, device="cuda").topk(k, -1).indices for _ in range(W)]).to(torch.int32)
    w_all = torch.rand(W, T, k, device="cuda") + 0.1
    row_src, row_dst, row_w, blk, _ = ep_row_tables(idx_all, w_all, 0, e_local)
    R = row_src.numel()
    stg = torch.empty(R, Hm, device="cuda", dtype=torch.bfloat16)
    fl = torch.empty(R // 128, device="cuda", dtype=torch.int32)
    cbufs = [torch.empty(k * T * Hm, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    hbox = [None]

    def dispatch():
        hbox[0] = o.gemm_grouped_dispatch(tab(xs), Hm, row_src, gate_up, blk, stg, fl, False)

    ms = timeit(dispatch, a.iters)
    report(f"MoE gate/up grouped GEMM with fused token dispatch R={R} N={2 * I} K={Hm} ({e_local} local experts)", ms, flops=2.0 * R * 2 * I * Hm)
    act = o.swiglu_fwd(hbox[0])
    ms = timeit(lambda: o.gemm_grouped_combine(act, down, blk, row_dst, row_w, tab(cbufs), Hm, False), a.iters)
    report(f"MoE down grouped GEMM with fused weighted combine R={R} N={Hm} K={I}", ms, flops=2.0 * R * Hm * I)
    torch.cuda.synchronize()
    _ext.check_status("fused_routed")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_layer", "layer_step", "gemm_fp8", "attn_fwd", "attn_bwd", "lmhead", "decode_attn", "elementwise", "fused_gather", "fused_emulated", "fused_routed", "all"])
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--ffn", type=int, default=18944)
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--sustained", action="store_true", help="layer_step: back-to-back launches for about a second instead of flushed single launches")
    ap.add_argument("--a-mn", dest="a_mn", action="store_true")
    ap.add_argument("--b-mn", dest="b_mn", action="store_true")
    ap.add_argument("--f32", action="store_true")
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--heads", type=int, default=28)
    ap.add_argument("--kv-heads", dest="kv_heads", type=int, default=4)
    ap.add_argument("--seqlen", type=int, default=1408)
    ap.add_argument("--batch", type=int, default=12)
    ap.add_argument("--vocab", type=int, default=152064)
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--impl", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    from verl_b200.ops import _ext

    _ext.load()
    if a.kernel in ("gemm", "all"):
        bench_gemm(a)
    if a.kernel == "gemm_layer":
        bench_gemm_layer(a)
    if a.kernel == "fused_routed":
        bench_fused_routed(a)
        return
    if a.kernel == "layer_step":
        bench_layer_step(a)
    if a.kernel in ("gemm_fp8", "all"):
        bench_gemm_fp8(a)
    if a.kernel == "fused_gather":
        bench_fused_gather(a)
    if a.kernel == "fused_emulated":
        bench_fused_emulated(a)
    if a.kernel in ("attn_fwd", "all"):
        bench_attn(a, False)
    if a.kernel in ("attn_bwd", "all"):
        bench_attn(a, True)
    if a.kernel in ("lmhead", "all"):
        a2 = argparse.Namespace(**vars(a))
        a2.m, a2.k = (a.m if a.kernel == "lmhead" else 4096), (a.k if a.kernel == "lmhead" else 3584)
        bench_lmhead(a2)
    if a.kernel in ("decode_attn", "all"):
        a2 = argparse.Namespace(**vars(a))
        if a.kernel == "all":
            a2.batch, a2.seqlen = 256, 900
        bench_decode_attn(a2)
    if a.kernel in ("elementwise", "all"):
        a2 = argparse.Namespace(**vars(a))
        if a.kernel == "all":
            a2.m, a2.k = 16384, 3584
        bench_elementwise(a2)
    _ext.check_status("kernel_bench")


if __name__ == "__main__":
    main()
