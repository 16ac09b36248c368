"""Timing of the fused compute+collective kernels against their NCCL(+cuBLAS) formulation, with roofline fractions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m verl_b200.parallel.comm_bench [--tokens 8192]

Every number is CUDA-event time on the launching stream after warm-up, MAX over ranks, with a buffer larger than L2
written between iterations. For each path the roofline time is the slower of (FLOPs ÷ measured bf16 GEMM peak) and
(bytes that must cross NVLink per GPU ÷ 770 GB/s, the measured peer-copy bandwidth per direction); the fused kernel and
the NCCL baseline are both reported as roofline ÷ achieved. Shapes are those of a Qwen2.5-7B layer.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "of measured"
    return 1590.0, 6650.0, "of fallback"


class Timer:
    def __init__(self):
        self.flush = torch.empty(64 * 1024 * 1024, device="cuda", dtype=torch.float32)

    def __call__(self, fn, iters=8, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ts = []
        for _ in range(iters):
            self.flush.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)


def report(rank, name, ms_fused, ms_base, flops, link_bytes):
    tf, _, tag = peaks()
    t_c = flops / (tf * 1e12) * 1e3 if flops else 0.0
    t_l = link_bytes / (NVLINK_GBS * 1e9) * 1e3 if link_bytes else 0.0
    roof = max(t_c, t_l)
    if rank == 0:
        bound = "compute" if t_c >= t_l else "NVLink"
        print(f"{name}: fused {ms_fused * 1e3:.0f} us ({roof / ms_fused:.2f} of roofline, {bound}-bound {roof * 1e3:.0f} us {tag}) | "
              f"NCCL+GEMM {ms_base * 1e3:.0f} us ({roof / ms_base:.2f}) | speed-up {ms_base / ms_fused:.2f}x", flush=True)


def bench_moe(a, rank, world, host, timer):
    """One expert-parallel MoE layer forward and forward+backward: dispatch / combine inside the grouped GEMMs against the
    all-to-all formulation (NCCL all-to-all + the same grouped GEMMs). ``--tokens`` tokens per rank."""
    from verl_b200.ops.moe import FusedEPContext, moe_forward

    dev = torch.device("cuda")
    T, H, I, E, k = a.tokens, a.moe_hidden, a.moe_ffn, a.experts, a.top_k
    el = E // world
    torch.manual_seed(rank)
    x = (0.5 * torch.randn(T, H, device=dev)).bfloat16().requires_grad_(True)
    torch.manual_seed(0)
    router = (0.02 * torch.randn(E, H, device=dev)).bfloat16().requires_grad_(True)
    gu = (0.02 * torch.randn(E, 2 * I, H, device=dev)).bfloat16()[rank * el:(rank + 1) * el].contiguous().requires_grad_(True)
    dn = (0.02 * torch.randn(E, H, I, device=dev)).bfloat16()[rank * el:(rank + 1) * el].contiguous().requires_grad_(True)
    ctx = FusedEPContext(dist.group.WORLD, host, T, H, k)
    g = torch.randn(T, H, device=dev).bfloat16()

    def run(ep_ctx, backward):
        y, _ = moe_forward(x, router, gu, dn, k, True, ep_group=dist.group.WORLD, ep_ctx=ep_ctx)
        if backward:
            torch.autograd.grad(y, (x, router, gu, dn), g)
        return y

    with torch.no_grad():
        y_f, y_b = run(ctx, False).float(), run(None, False).float()
    err = ((y_f - y_b).abs().max() / y_b.abs().max()).item()
    # rows that leave the rank: (W-1)/W of T*k rows of H bf16, once for dispatch and once for combine
    link = 2.0 * T * k * H * 2 * (world - 1) / world
    flops = 2.0 * T * k * H * 3 * I
    with torch.no_grad():
        ms_f, ms_b = timer(lambda: run(ctx, False)), timer(lambda: run(None, False))
    report(rank, f"MoE layer forward, EP={world}, {T} tokens/rank, E={E} top-{k}, H={H} I={I} (max rel diff {err:.1e})", ms_f, ms_b, flops, link)
    ms_f, ms_b = timer(lambda: run(ctx, True)), timer(lambda: run(None, True))
    report(rank, "MoE layer forward + backward, same shapes", ms_f, ms_b, 3 * flops, 2 * link)
    # where the fused forward spends its time: the same steps, timed one by one
    from verl_b200.ops import _ext
    from verl_b200.ops.moe import GROUP_BLOCK, ep_row_tables, route_topk

    o = _ext.ops()
    with torch.no_grad():
        logits = torch.nn.functional.linear(x, router)
        w, idx, _ = route_topk(logits, k, True)
        t_route = timer(lambda: route_topk(torch.nn.functional.linear(x, router), k, True))

        def gather_routing():
            idx_all = torch.empty(world, T, k, dtype=torch.int32, device=dev)
            w_all = torch.empty(world, T, k, dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(idx_all, idx.to(torch.int32).contiguous())
            dist.all_gather_into_tensor(w_all, w.float().contiguous())
            return idx_all, w_all

        idx_all, w_all = gather_routing()
        t_gather = timer(gather_routing)
        t_tables = timer(lambda: ep_row_tables(idx_all.long(), w_all, rank, el))
        row_src, row_dst, row_w, blk, rng = ep_row_tables(idx_all.long(), w_all, rank, el)
        R = row_src.numel()
        t_publish = timer(lambda: ctx.publish(x.detach()))
        xg = torch.empty(R, H, dtype=torch.bfloat16, device=dev)
        flags = torch.empty(R // GROUP_BLOCK, dtype=torch.int32, device=dev)
        h = o.gemm_grouped_dispatch(ctx.xbuf.table(), H, row_src, gu.detach(), blk, xg, flags, False)
        t_dispatch = timer(lambda: o.gemm_grouped_dispatch(ctx.xbuf.table(), H, row_src, gu.detach(), blk, xg, flags, False))
        t_plain = timer(lambda: o.gemm_grouped(xg, gu.detach(), blk, False))
        a_ = o.swiglu_fwd(h)
        t_act = timer(lambda: o.swiglu_fwd(h))
        t_combine = timer(lambda: o.gemm_grouped_combine(a_, dn.detach(), blk, row_dst, row_w, ctx.cbuf.table(), H, False))
        t_plain2 = timer(lambda: o.gemm_grouped(a_, dn.detach(), blk, False))
        t_collect = timer(lambda: ctx.collect(T, T))
    if rank == 0:
        print(f"  fused forward by step (us, R = {R} rows): router {t_route * 1e3:.0f} | routing all-gather {t_gather * 1e3:.0f} | row tables {t_tables * 1e3:.0f} | "
              f"publish + barrier {t_publish * 1e3:.0f} | dispatch GEMM {t_dispatch * 1e3:.0f} (same GEMM on local rows {t_plain * 1e3:.0f}) | swiglu {t_act * 1e3:.0f} | "
              f"combine GEMM {t_combine * 1e3:.0f} (plain {t_plain2 * 1e3:.0f}) | barrier + slot sum {t_collect * 1e3:.0f}", flush=True)


def bench_decode(a, rank, world, host, timer):
    """The two row-parallel projections of a decode step (256 sequences) as GEMM -> all-reduce, every split-K choice next to the
    plan's own, against cuBLAS + NCCL: attention output projection (K = heads x 128 / W) and MLP down projection (K = ffn / W)."""
    from verl_b200.ops import _ext
    from verl_b200.parallel.tp import TPContext

    o = _ext.ops()
    H, F, W = a.hidden, a.ffn, world
    dev = torch.device("cuda")
    ctx = TPContext(dist.group.WORLD, host, max_tokens=512, hidden=H, max_out=H)
    for name, K in (("down projection", F // W), ("output projection", H // W)):
        x = torch.randn(256, K, device=dev).bfloat16()
        w = (0.02 * torch.randn(H, K, device=dev)).bfloat16()
        os.environ["VERL_B200_COMM"] = "nccl"
        ms_b = timer(lambda: ctx.gemm_allreduce(x, w))
        os.environ["VERL_B200_COMM"] = "native"
        ms_f = timer(lambda: ctx.gemm_allreduce(x, w))
        report(rank, f"decode GEMM -> all-reduce, {name} [256x{K}] x [{H}x{K}]^T, TP={W}, planned split", ms_f, ms_b, 2.0 * 256 * H * K, (W - 1) * 256 * H * 2)
        out = torch.empty(256, H, dtype=torch.bfloat16, device=dev)
        for bn, sk in ((256, 5), (256, 3), (256, 2), (128, 4), (128, 2), (128, 1), (64, 2), (64, 1)):
            if (K // 64) // sk < 8:
                continue
            ms = timer(lambda: o.gemm_allreduce_sig(x, w, ctx.slots2.table(), ctx.sig.table(), ctx.rank, ctx.half_elems, ctx.slots2.tensor(torch.bfloat16),
                                                    ctx.sig.tensor(torch.int32, 64), None, out, bn, sk))
            if rank == 0:
                print(f"    tile N = {bn}, K slices = {sk}: {ms * 1e3:.1f} us", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=3584)
    ap.add_argument("--ffn", type=int, default=18944)
    ap.add_argument("--params-m", type=int, default=512, help="millions of parameters for the optimizer-step paths")
    ap.add_argument("--only", default="", help="'moe': only the expert-parallel MoE layer (Qwen3-30B-A3B shapes); 'decode': only the decode-size GEMM -> all-reduce pairs with a split-K sweep")
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--top-k", dest="top_k", type=int, default=8)
    ap.add_argument("--moe-hidden", dest="moe_hidden", type=int, default=2048)
    ap.add_argument("--moe-ffn", dest="moe_ffn", type=int, default=768)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("cpu:gloo,cuda:nccl")
    from verl_b200.ops import _ext
    from verl_b200.parallel.symm_mem import SymmetricBuffer
    from verl_b200.parallel.tp import TPContext
    from verl_b200.single_controller.spmd import init_spmd_process_group

    host = init_spmd_process_group()
    o = _ext.ops()
    dev = torch.device("cuda")
    timer = Timer()
    T, H, F = a.tokens, a.hidden, a.ffn
    torch.manual_seed(0)
    W = world
    if a.only == "moe":
        bench_moe(a, rank, world, host, timer)
        dist.barrier()
        dist.destroy_process_group()
        return
    if a.only == "decode":
        bench_decode(a, rank, world, host, timer)
        dist.barrier()
        dist.destroy_process_group()
        return

    # ---- 1. sharded optimizer step: reduce-scatter(+scale, +sum g^2) and AdamW(+all-gather)
    n = a.params_m * 1_000_000 // (W * 1024) * (W * 1024)
    shard = n // W
    g_sym = SymmetricBuffer(n * 4, host_group=host)
    p_sym = SymmetricBuffer(n * 2, host_group=host)
    g_sym.tensor(torch.float32, n).normal_()
    out = torch.empty(shard, device=dev)
    sumsq = torch.zeros(1, device=dev)
    g_sym.barrier()
    g_plain = torch.randn(n, device=dev)

    def rs_fused():
        o.symm_reduce_scatter(g_sym.table(), W, rank * shard, out, sumsq, 1.0 / W)

    def rs_nccl():
        dist.reduce_scatter_tensor(out, g_plain, op=dist.ReduceOp.AVG)
        sumsq.copy_(out.float().pow(2).sum())

    ms_f, ms_b = timer(rs_fused), timer(rs_nccl)
    report(rank, f"grad reduce-scatter + 1/W + sum g^2, {n / 1e6:.0f} M fp32, W={W}", ms_f, ms_b, 0, (W - 1) * shard * 4)
    master, m1, m2 = torch.randn(shard, device=dev), torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
    scal = torch.tensor([1.0, 0.0, 0.0, 0.0], device=dev)
    flat = torch.empty(n, device=dev, dtype=torch.bfloat16)

    def ag_fused():
        o.symm_adamw_allgather(master, m1, m2, out, p_sym.table(), W, rank * shard, 1e-6, 0.9, 0.999, 1e-8, 0.01, 1, scal)

    def ag_nccl():
        o.adamw_(master, m1, m2, out, flat[rank * shard:(rank + 1) * shard], 1e-6, 0.9, 0.999, 1e-8, 0.01, 1, scal)
        dist.all_gather_into_tensor(flat, flat[rank * shard:(rank + 1) * shard].clone())

    ms_f, ms_b = timer(ag_fused), timer(ag_nccl)
    report(rank, f"AdamW + bf16 all-gather, {n / 1e6:.0f} M params, W={W}", ms_f, ms_b, 0, (W - 1) * shard * 2)
    p_sym.barrier()

    # ---- 2. tensor-parallel GEMMs of one layer (column-parallel up-projection, row-parallel down-projection)
    Tl = T // W
    ctx = TPContext(dist.group.WORLD, host, max_tokens=T, hidden=H, max_out=H)
    x_shard = torch.randn(Tl, H, device=dev).bfloat16()
    w_up = (0.02 * torch.randn(2 * F // W, H, device=dev)).bfloat16()
    os.environ["VERL_B200_COMM"] = "native"
    ms_f = timer(lambda: ctx.allgather_linear(x_shard, w_up))
    os.environ["VERL_B200_COMM"] = "nccl"
    ms_b = timer(lambda: ctx.allgather_linear(x_shard, w_up))
    report(rank, f"all-gather -> GEMM  [{T}x{H}] x [{2 * F // W}x{H}]^T, TP={W}", ms_f, ms_b, 2.0 * T * H * (2 * F // W), (W - 1) * Tl * H * 2)
    x_mid = torch.randn(T, F // W, device=dev).bfloat16()
    w_dn = (0.02 * torch.randn(H, F // W, device=dev)).bfloat16()
    os.environ["VERL_B200_COMM"] = "native"
    ms_f = timer(lambda: ctx.gemm_reduce_scatter(x_mid, w_dn))
    os.environ["VERL_B200_COMM"] = "nccl"
    ms_b = timer(lambda: ctx.gemm_reduce_scatter(x_mid, w_dn))
    report(rank, f"GEMM -> reduce-scatter  [{T}x{F // W}] x [{H}x{F // W}]^T, TP={W}", ms_f, ms_b, 2.0 * T * H * (F // W), (W - 1) * Tl * H * 2)
    x_dec = torch.randn(256, F // W, device=dev).bfloat16()
    os.environ["VERL_B200_COMM"] = "native"
    ms_f = timer(lambda: ctx.gemm_allreduce(x_dec, w_dn))
    os.environ["VERL_B200_COMM"] = "nccl"
    ms_b = timer(lambda: ctx.gemm_allreduce(x_dec, w_dn))
    report(rank, f"GEMM -> all-reduce (decode, 256 tokens) [{256}x{F // W}] x [{H}x{F // W}]^T, TP={W}", ms_f, ms_b, 2.0 * 256 * H * (F // W), (W - 1) * 256 * H * 2)
    os.environ["VERL_B200_COMM"] = "native"
    ctx.allreduce_mode = "barrier"
    ms_f2 = timer(lambda: ctx.gemm_allreduce(x_dec, w_dn))
    ctx.allreduce_mode = "signal"
    report(rank, "  same, four-launch variant (GEMM, barrier, slot sum, barrier)", ms_f2, ms_b, 2.0 * 256 * H * (F // W), (W - 1) * 256 * H * 2)

    # ---- 3. ZeRO-3 style weight gather fused into the GEMM
    ws = SymmetricBuffer((2 * F // W) * H * 2, host_group=host)
    ws.tensor(torch.bfloat16).view(2 * F // W, H).normal_(0, 0.02)
    ws.barrier()
    x_full = torch.randn(T, H, device=dev).bfloat16()
    w_full = torch.empty(2 * F, H, device=dev, dtype=torch.bfloat16)
    w_loc = ws.tensor(torch.bfloat16).view(2 * F // W, H)

    def wg_nccl():
        dist.all_gather_into_tensor(w_full, w_loc)
        torch.nn.functional.linear(x_full, w_full)

    w_stage = torch.empty(2 * F * H, device=dev, dtype=torch.bfloat16)
    w_flags = torch.zeros(2 * F // 128 + 8, device=dev, dtype=torch.int32)
    ep = [0]

    def wg_fused():
        ep[0] += 1
        return TPContext.weight_gather_linear(x_full, ws, 2 * F // W, H, 0, w_stage, w_flags, ep[0])

    ms_f = timer(wg_fused)
    ms_b = timer(wg_nccl)
    report(rank, f"weight all-gather -> GEMM  [{T}x{H}] x [{2 * F}x{H}]^T, shards={W}", ms_f, ms_b, 2.0 * T * H * 2 * F, (W - 1) * (2 * F // W) * H * 2)
    ws.barrier()

    # ---- 4. Ulysses: sequence<->head all-to-all fused into the projections (needs heads divisible by W)
    from verl_b200.models.config import PRESETS
    from verl_b200.parallel.ulysses import FusedUlysses, _a2a, fused_ulysses_available

    cfg = PRESETS["qwen2.5-7b"]
    if fused_ulysses_available(x_shard, cfg, W):
        fu = FusedUlysses(dist.group.WORLD, host, cfg, T)
        D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        w_qkv = (0.02 * torch.randn((Hq + 2 * Hkv) * D, H, device=dev)).bfloat16()
        b_qkv = torch.zeros((Hq + 2 * Hkv) * D, device=dev, dtype=torch.bfloat16)

        def qkv_nccl():
            y = torch.nn.functional.linear(x_shard, w_qkv, b_qkv)
            q, k, v = y.split([Hq * D, Hkv * D, Hkv * D], -1)
            return [_a2a(t.reshape(Tl, -1, D), 1, 0, dist.group.WORLD) for t in (q, k, v)]

        ms_f, ms_b = timer(lambda: fu.qkv_forward(x_shard, w_qkv, b_qkv)), timer(qkv_nccl)
        report(rank, f"QKV projection + seq->head all-to-all, {Tl} local tokens, SP={W}", ms_f, ms_b, 2.0 * Tl * H * (Hq + 2 * Hkv) * D,
               (W - 1) * Tl * (Hq + 2 * Hkv) * D * 2 // W)
        o_loc = torch.randn(T, fu.Kl, device=dev).bfloat16()
        w_o = (0.02 * torch.randn(H, Hq * D, device=dev)).bfloat16()

        def o_nccl():
            t = _a2a(o_loc.reshape(T, -1, D), 0, 1, dist.group.WORLD).reshape(Tl, Hq * D)
            return torch.nn.functional.linear(t, w_o)

        ms_f, ms_b = timer(lambda: fu.o_forward(o_loc, w_o, Tl)), timer(o_nccl)
        report(rank, f"head->seq all-to-all + output projection, {Tl} local tokens, SP={W}", ms_f, ms_b, 2.0 * Tl * H * Hq * D,
               (W - 1) * Tl * Hq * D * 2 // W)
        # forward + backward of both projections: the backward routes d(attention output) through the scatter epilogue and
        # gathers d(qkv) inside the activation-gradient GEMM; the baseline keeps the fused forward and uses all-to-alls in backward
        from verl_b200.parallel.ulysses import _FusedOProj, _FusedQKV

        wq_p, wo_p = torch.nn.Parameter(w_qkv.clone()), torch.nn.Parameter(w_o.clone())
        for p_ in (wq_p, wo_p):
            p_.main_grad = torch.zeros(p_.shape, device=dev, dtype=torch.float32)
        g_qkv = torch.randn(T, fu.Cl, device=dev).bfloat16()
        g_out = torch.randn(Tl, H, device=dev).bfloat16()

        def sp_fb(fused_bwd):
            fu.fused_backward = fused_bwd
            xs = x_shard.clone().requires_grad_(True)
            _FusedQKV.apply(xs, wq_p, None, fu).backward(g_qkv)
            ol = o_loc.clone().requires_grad_(True)
            _FusedOProj.apply(ol, wo_p, fu, Tl).backward(g_out)

        ms_f, ms_b = timer(lambda: sp_fb(True)), timer(lambda: sp_fb(False))
        fu.fused_backward = True
        report(rank, f"Ulysses QKV + output projection, forward + backward, {Tl} local tokens, SP={W} (baseline: fused forward, all-to-all backward)",
               ms_f, ms_b, 6.0 * Tl * H * (2 * Hq + 2 * Hkv) * D, 2 * (W - 1) * Tl * (2 * Hq + 2 * Hkv) * D * 2 // W)
    elif rank == 0:
        print(f"Ulysses paths skipped: {cfg.num_key_value_heads} KV heads do not divide by SP={W}")

    # ---- 5. sequence-parallel TP block (column-parallel then row-parallel projection), forward + backward through autograd:
    # backward = activation-gradient GEMM -> reduce-scatter epilogue (column-parallel) and all-gather -> activation-gradient GEMM
    # whose staged operand also feeds the weight gradient (row-parallel)
    from verl_b200.parallel.tp import allgather_linear, linear_reduce_scatter

    w1 = torch.nn.Parameter((0.02 * torch.randn(F // W, H, device=dev)).bfloat16())
    w2 = torch.nn.Parameter((0.02 * torch.randn(H, F // W, device=dev)).bfloat16())
    for p_ in (w1, w2):
        p_.main_grad = torch.zeros(p_.shape, device=dev, dtype=torch.float32)
    g_sh = torch.randn(Tl, H, device=dev).bfloat16()

    def tp_fb(env):
        os.environ["VERL_B200_COMM"] = env
        xs = x_shard.clone().requires_grad_(True)
        y = allgather_linear(xs, w1, None, dist.group.WORLD, ctx)
        linear_reduce_scatter(y, w2, dist.group.WORLD, ctx).backward(g_sh)

    ms_f, ms_b = timer(lambda: tp_fb("native")), timer(lambda: tp_fb("nccl"))
    os.environ["VERL_B200_COMM"] = "native"
    report(rank, f"sequence-parallel TP block [{T}x{H}] -> {F // W} -> {H}, forward + backward, TP={W}", ms_f, ms_b, 6.0 * T * H * (F // W) * 2,
           4 * (W - 1) * Tl * H * 2)
    torch.cuda.synchronize()
    _ext.check_status("comm_bench")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
