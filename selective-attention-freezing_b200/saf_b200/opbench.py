"""Operator timings on the benchmark shapes: each operator of the hot path, forward and backward, launched
alone on seeded synthetic tensors and timed with CUDA events (median).  The counterpart of the reference's
per-operator probes (qwen/nanogpt/bench_qwen_prefill_triton.py:186-225); also the command the ncu captures
of single kernels are taken from.

    python -m saf_b200.opbench --workload c3 --ops attn_fwd,attn_bwd,qk_fwd,qk_bwd,layer_infer,layer_train \
                               [--B 2 --T 8192] [--reps 5] [--frozen sink_decay|dense|decomposed|none]
                               [--impl ours|ref-triton|sdpa-flash|sdpa-cudnn]

--impl times the same attention call (attn_fwd / attn_bwd) through another implementation on the same box with the
same CUDA-event protocol: `ref-triton` = the reference's own Triton `fused_mixed_attn` (kernel/fused_attn.py:650-734;
qwen/kernel/fused_attn.py for grouped-query shapes), loaded from the checkout named by SAF_REFERENCE_ROOT, with the
frozen heads' patterns stored densely as the reference must hold them; `sdpa-flash` / `sdpa-cudnn` = torch's
scaled_dot_product_attention on the live heads only, restricted to that backend.

Prints one JSON line per operator: ms, algorithmic TFLOP/s (backward counted as 2.5x / 2x the forward
FLOPs, as the reference's roofline does) and the library launches of one call.
"""
import argparse
import json
import os
import sys

import torch

if __package__ in (None, ""):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from saf_b200 import ops, synthetic  # noqa: E402


def _timed(fn, reps):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2]


def _load_reference_kernel(gqa):
    """The reference's kernel package under a private module name (this process already owns `kernel`)."""
    import importlib.util
    root = os.environ.get("SAF_REFERENCE_ROOT")
    if not root:
        raise SystemExit("--impl ref-triton needs SAF_REFERENCE_ROOT (a checkout of the reference project)")
    pkg_dir = os.path.join(root, "qwen", "kernel") if gqa else os.path.join(root, "kernel")
    name = "saf_reference_kernel_gqa" if gqa else "saf_reference_kernel"
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _other_attention(impl, q, k, v, patt, frozen, hidx, kw, fz, live, T, gqa):
    """The same attention call through the reference's Triton kernel or torch SDPA (live heads only)."""
    dev = q.device
    H = frozen.numel()
    if impl == "ref-triton":
        ref = _load_reference_kernel(gqa)
        rkw = {n: t for n, t in kw.items() if n in ("alpha", "rho", "z", "pidx", "kvidx")}
        rfrozen, rpatt = frozen, patt
        if "sink_decay" in kw:
            # the reference can hold this pattern family only as dense stored planes (state 1)
            a, r = kw["sink_decay"]
            planes = []
            for h in fz:
                pl = torch.empty(T, T, device=dev, dtype=torch.bfloat16)
                for i0 in range(0, T, 2048):
                    i = torch.arange(i0, min(i0 + 2048, T), device=dev, dtype=torch.float64)[:, None]
                    j = torch.arange(T, device=dev, dtype=torch.float64)[None, :]
                    dec = torch.where(i >= j, r[h].double() ** (i - j).clamp(min=0), torch.zeros((), device=dev, dtype=torch.float64))
                    dec = dec / dec.sum(-1, keepdim=True) * (1.0 - a[h].double())
                    dec[:, 0] += a[h].double()
                    pl[i0:i0 + 2048] = dec.to(torch.bfloat16)
                planes.append(pl)
            rpatt = torch.stack(planes)
            pidx = torch.zeros(H, dtype=torch.int32)
            for s_, h in enumerate(fz):
                pidx[h] = s_
            rkw["pidx"] = pidx.to(dev)
            rfrozen = (frozen != 0).to(torch.int32)
        if "alpha" in rkw:
            rkw["rho_band"] = ref.make_rho_band(rkw["rho"])
        return lambda: ref.fused_mixed_attn(q, k, v, rpatt, rfrozen, hidx, validate=False, **rkw)
    from torch.nn.attention import SDPBackend, sdpa_kernel
    backend = SDPBackend.FLASH_ATTENTION if impl == "sdpa-flash" else SDPBackend.CUDNN_ATTENTION
    li = torch.tensor(live, device=dev)
    if gqa:
        kvh = kw["kvidx"].long()[li]
        kk, vv = k.detach()[:, kvh].contiguous(), v.detach()[:, kvh].contiguous()
    else:
        kk, vv = k, v.detach()[:, li].contiguous().requires_grad_(v.requires_grad)

    def run():
        with sdpa_kernel([backend]):
            out = torch.nn.functional.scaled_dot_product_attention(q, kk, vv, is_causal=True)
        return out
    run.live_only = True
    return run


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--ops", default="attn_fwd,attn_bwd,qk_fwd,qk_bwd")
    ap.add_argument("--B", type=int, default=None)
    ap.add_argument("--T", type=int, default=None)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--frozen", default="sink_decay", choices=["sink_decay", "dense", "decomposed", "none"])
    ap.add_argument("--impl", default="ours", choices=["ours", "ref-triton", "sdpa-flash", "sdpa-cudnn"])
    ap.add_argument("--trace", action="store_true",
                    help="after the runs, print the per-step clock stamps a library built with -DSAF_FWD_TRACE / "
                         "-DSAF_BWD_TRACE recorded for one CTA (heaviest tile of batch 0, head 0; head 0 must be live)")
    args = ap.parse_args()
    if "mma_rate" in args.ops.split(","):
        return print_mma_rate()
    w = dict(synthetic.WORKLOADS[args.workload])
    if args.B:
        w["B"] = args.B
    if args.T:
        w["T"] = args.T
    dev = torch.device("cuda")
    B, T, H, hd, nf = w["B"], w["T"], w["n_head"], w["head_dim"], w["n_frozen"]
    if args.frozen == "none":
        nf = 0
    C, U = H * hd, H - nf
    fz = synthetic.frozen_heads_for_layer(H, nf, 1337, 0) if nf else []
    live = [h for h in range(H) if h not in fz]
    g = torch.Generator().manual_seed(7)
    state = {"sink_decay": 3, "dense": 1, "decomposed": 2, "none": 0}[args.frozen]
    frozen = torch.tensor([state if h in fz else 0 for h in range(H)], dtype=torch.int32, device=dev)
    hidx = torch.zeros(H, dtype=torch.int32)
    for s, h in enumerate(live):
        hidx[h] = s
    hidx = hidx.to(dev)
    n_kv = w.get("n_kv")
    gqa = n_kv is not None          # q head h reads K/V head kvidx[h]; forward only, as in the reference
    q = torch.randn(B, U, T, hd, generator=g).bfloat16().to(dev).requires_grad_(not gqa)
    k = torch.randn(B, n_kv if gqa else U, T, hd, generator=g).bfloat16().to(dev).requires_grad_(not gqa)
    v = torch.randn(B, n_kv if gqa else H, T, hd, generator=g).bfloat16().to(dev).requires_grad_(not gqa)
    dy = torch.randn(B, H, T, hd, generator=g).bfloat16().to(dev)
    kw, patt = {}, None
    if gqa:
        kw["kvidx"] = torch.tensor([h * n_kv // H for h in range(H)], dtype=torch.int32, device=dev)
    if nf and args.frozen == "sink_decay":
        a, r = synthetic.sink_decay_params(H, 2337)
        kw["sink_decay"] = (a.float().to(dev), r.float().to(dev))
    elif nf and args.frozen == "decomposed":
        alpha = (torch.randn(H, T, generator=g) * 0.5).to(dev)
        rho = (-0.002 * torch.arange(T).float()[None] + torch.randn(H, T, generator=g) * 0.3).to(dev)
        kw.update(alpha=alpha, rho=rho, z=ops.decomposed_logz(alpha, rho))
    elif nf:
        p = torch.rand(nf, T, T, generator=g).tril_()
        patt = (p / p.sum(-1, keepdim=True)).bfloat16().to(dev)
        pidx = torch.zeros(H, dtype=torch.int32)
        for s, h in enumerate(fz):
            pidx[h] = s
        kw["pidx"] = pidx.to(dev)
    x = torch.randn(B, T, C, generator=g).bfloat16().to(dev).requires_grad_(True)
    w1 = (torch.randn(C, C, generator=g) * 0.02).bfloat16().to(dev).requires_grad_(True)
    w2 = (torch.randn(C, C, generator=g) * 0.02).bfloat16().to(dev).requires_grad_(True)
    rows = (torch.tensor(live)[:, None] * hd + torch.arange(hd)).reshape(-1).to(dev)
    cos, sin = synthetic.rope_tables(hd, T, base=w["rope_base"], device=dev)
    dqk = torch.randn(B, T, 2 * U * hd, generator=g).bfloat16().to(dev)

    def attn():
        return ops.fused_mixed_attn(q, k, v, patt, frozen, hidx, validate=False, **kw)

    if args.impl != "ours":
        attn = _other_attention(args.impl, q, k, v, patt, frozen, hidx, kw, fz, live, T, gqa)

    def qk():
        return ops.linear_rows2(x, w1, w2, None, None, rows, rope=(cos, sin), head_dim=hd)

    fl_attn = 2.0 * B * U * T * T * hd
    fl_qk = 2.0 * B * T * C * 2 * U * hd
    shape = f"B{B} T{T} H{H}{'/kv%d' % n_kv if gqa else ''} hd{hd} live{U} frozen{nf}({args.frozen})"
    for op in args.ops.split(","):
        extra = {}
        if op == "attn_fwd":
            with torch.no_grad():
                n0 = ops.launch_count()
                attn()
                n = ops.launch_count() - n0
                ms = _timed(attn, args.reps)
            fl = fl_attn
        elif op == "attn_bwd":
            y = attn()
            gy = dy[:, live].contiguous() if getattr(attn, "live_only", False) else dy
            n0 = ops.launch_count()
            y.backward(gy, retain_graph=True)
            n = ops.launch_count() - n0

            def run():
                q.grad = k.grad = v.grad = None
                y.backward(gy, retain_graph=True)
            ms = _timed(run, args.reps)
            fl = 2.5 * fl_attn
        elif op == "qk_fwd":
            with torch.no_grad():
                n0 = ops.launch_count()
                qk()
                n = ops.launch_count() - n0
                ms = _timed(qk, args.reps)
            fl = fl_qk
        elif op == "qk_bwd":
            y = qk()
            n0 = ops.launch_count()
            y.backward(dqk, retain_graph=True)
            n = ops.launch_count() - n0

            def run():
                x.grad = w1.grad = w2.grad = None
                y.backward(dqk, retain_graph=True)
            ms = _timed(run, args.reps)
            fl = 2.0 * fl_qk
        elif op in ("frozen_pv", "frozen_pv_bwd"):
            # the frozen heads alone through frozen_pv: scan for sink+decay patterns (HBM-bound: V read + Y written),
            # lower-triangular GEMM for dense stored ones
            assert nf and args.frozen in ("sink_decay", "dense"), "frozen_pv needs --frozen sink_decay or dense"
            vf = v.detach()[:, fz].contiguous().requires_grad_(op == "frozen_pv_bwd")
            if args.frozen == "sink_decay":
                sd = (kw["sink_decay"][0][fz].contiguous(), kw["sink_decay"][1][fz].contiguous())

                def fpv():
                    return ops.frozen_pv(None, vf, None, T, sink_decay=sd)
            else:
                fidx = torch.arange(nf, dtype=torch.int32, device=dev)

                def fpv():
                    return ops.frozen_pv(patt, vf, fidx, T)
            if op == "frozen_pv":
                with torch.no_grad():
                    n0 = ops.launch_count()
                    fpv()
                    n = ops.launch_count() - n0
                    ms = _timed(fpv, args.reps)
            else:
                yf = fpv()
                dyf = dy[:, fz].contiguous()
                n0 = ops.launch_count()
                yf.backward(dyf, retain_graph=True)
                n = ops.launch_count() - n0

                def run():
                    vf.grad = None
                    yf.backward(dyf, retain_graph=True)
                ms = _timed(run, args.reps)
            fl = 1.0 * B * nf * T * T * hd if args.frozen == "dense" else 0.0
            extra["gbs"] = round(B * nf * T * hd * 2 * 2 / ms / 1e6, 1)      # values read + result written
        elif op == "pattern_grad":
            # parameter gradients of the decomposed heads (needs --frozen decomposed): dS = P (dO V^T - delta)
            from saf_b200.trainable_patterns import pattern_param_grad
            assert nf and args.frozen == "decomposed", "pattern_grad needs --frozen decomposed"
            with torch.no_grad():
                y = attn()

                def run():
                    return pattern_param_grad(dy, y, v, kw["alpha"], kw["rho"], kw["z"], frozen)
                n0 = ops.launch_count()
                run()
                n = ops.launch_count() - n0
                ms = _timed(run, args.reps)
            fl = 1.0 * B * nf * T * T * hd          # causal half of 2 T^2 hd per head
        elif op == "attn_stats":
            # controller statistics of the live heads (flash forward for the row lse + the statistics kernel);
            # the running mean is (U, T, T) fp32 on the device
            from saf_b200.capture import AttentionMoments
            acc = AttentionMoments(U, T, dev)
            qd, kd = q.detach(), k.detach()
            with torch.no_grad():
                acc.update(qd, kd)                  # first batch: plain write of the mean
                n0 = ops.launch_count()
                acc.update(qd, kd)                  # later batches: read-merge-write
                n = ops.launch_count() - n0
                ms = _timed(lambda: acc.update(qd, kd), args.reps)
            fl = 1.5 * fl_attn                      # the lse pass (QK^T and PV) + QK^T again
            del acc
        elif op in ("layer_train", "layer_infer"):
            # the whole attention module (projections + mixed attention + c_proj) at this shape
            from types import SimpleNamespace
            from saf_b200.attention import SafCausalSelfAttention
            cfg = SimpleNamespace(n_embd=C, n_head=H, block_size=T, bias=False, dropout=0.0, position_encoding="rope",
                                  rand_attn_prior_repr="dense", freeze_pattern_dtype="bfloat16")
            m = SafCausalSelfAttention(cfg).to(dev)
            if nf:
                a_, r_ = synthetic.sink_decay_params(nf, 2337)
                m.freeze_heads_sink_decay(fz, a_.tolist(), r_.tolist())
            rope = (cos.view(1, 1, T, hd), sin.view(1, 1, T, hd))
            if op == "layer_infer":
                m = m.bfloat16().eval()
                xi = x.detach()

                def run():
                    with torch.inference_mode():
                        m(xi, rope=rope)
                fl = fl_attn + 2.0 * B * T * C * (2 * U + 2 * H) * hd
            else:
                xi = x.detach().float().requires_grad_(True)     # fp32 master weights, bf16 autocast

                def run():
                    xi.grad = None
                    for prm in m.parameters():
                        prm.grad = None
                    with torch.autocast("cuda", dtype=torch.bfloat16):
                        out = m(xi, rope=rope)
                    out.backward(dy.transpose(1, 2).reshape(B, T, C).to(out.dtype))
                fl = 3.5 * fl_attn + 3 * 2.0 * B * T * C * (2 * U + 2 * H) * hd
            n0 = ops.launch_count()
            run()
            n = ops.launch_count() - n0
            ms = _timed(run, args.reps)
        elif op in ("block_infer", "mlp_infer"):
            # whole transformer block (LayerNorms, attention path, MLP with fused epilogues) or its MLP half
            from types import SimpleNamespace
            from saf_b200.block import SafBlock
            cfg = SimpleNamespace(n_embd=C, n_head=H, block_size=T, bias=False, dropout=0.0, position_encoding="rope",
                                  rand_attn_prior_repr="dense", freeze_pattern_dtype="bfloat16")
            blk = SafBlock(cfg).to(dev)
            if nf:
                a_, r_ = synthetic.sink_decay_params(nf, 2337)
                blk.main_block.freeze_heads_sink_decay(fz, a_.tolist(), r_.tolist())
            blk = blk.bfloat16().eval()
            rope = (cos.view(1, 1, T, hd), sin.view(1, 1, T, hd))
            xi = x.detach()
            fl_mlp = 2.0 * B * T * C * 8 * C
            if op == "block_infer":
                def run():
                    with torch.inference_mode():
                        blk(xi, rope=rope)
                fl = fl_attn + 2.0 * B * T * C * (2 * U + 2 * H) * hd + fl_mlp
            else:
                def run():
                    with torch.inference_mode():
                        blk.mlp(blk.ln_2(xi), residual=xi)
                fl = fl_mlp
            n0 = ops.launch_count()
            run()
            n = ops.launch_count() - n0
            ms = _timed(run, args.reps)
        else:
            raise SystemExit("unknown op %r" % op)
        print(json.dumps({"op": op, "impl": args.impl, "shape": shape, "ms": round(ms, 4),
                          "tflops": round(fl / ms / 1e9, 1), "launches": n, **extra}), flush=True)


# (what is issued, tensor-pipe cycles per instruction at 4096 multiply-adds per clock, instructions per group)
MMA_FORMS = (
    ("A smem K-major, B smem K-major, N 128", 64.0, 8),
    ("A TMEM, B smem MN-major, N 128", 64.0, 8),
    ("A TMEM, B smem MN-major, N 64", 32.0, 8),
    ("A smem MN-major, B smem MN-major, N 256", 128.0, 8),
    ("A smem K-major, B smem K-major, N 256", 128.0, 8),
    ("A TMEM, B smem K-major, N 128", 64.0, 8),
    ("A smem K-major, B smem K-major, N 64", 32.0, 8),
    ("A smem K-major, B smem MN-major, N 128", 64.0, 8),
    ("ring stages, descriptors built per instruction: A smem, B smem K-major, N 128", 64.0, 8),
    ("ring stages, descriptors built per instruction: A TMEM, B smem MN-major, N 128", 64.0, 8),
    ("ring stages, descriptors advanced by an add: A smem, B smem K-major, N 128", 64.0, 8),
    ("ring stages, descriptors advanced by an add: A TMEM, B smem MN-major, N 128", 64.0, 8),
    ("a new product every 8 instructions, two accumulators in turn, commit after each: smem operands, N 128", 64.0, 8),
    ("a new product every 8 instructions, two accumulators in turn, no commits: smem operands, N 128", 64.0, 8),
    ("smem-operand and TMEM-operand products in turn (TMEM operand in columns 0-31 and 64-95 of its region), N 128", 64.0, 8),
    ("a new product every 8 instructions, one accumulator, commit after each: smem operands, N 128", 64.0, 8),
    ("forward key step hd 64, all operands from TMEM: 4 score + 4 P V instructions of N 64 in turn", 32.0, 4),
    ("forward key step hd 64: 4 score instructions N 128 from smem, 8 P V instructions N 64 from TMEM, in turn",
     512.0 / 12, 6),
    ("forward key step hd 64: the same, issued score, score, P V, P V", 512.0 / 12, 6),
    ("smem- and TMEM-operand products in turn, the TMEM-operand one as two halves of N 64 (8 + 16 instructions)",
     1024.0 / 24, 12),
    ("smem- and TMEM-operand products in turn, the TMEM-operand one with a K-major B operand, N 128", 64.0, 8),
    ("smem- and TMEM-operand products in turn, the TMEM operand in consecutive columns, N 128", 64.0, 8),
)


def print_mma_rate(reps=2048):
    """Cycles per tcgen05.mma instruction (bf16, M 128, K 16) for the operand forms the kernels use
    (`saf_selftest_mma_rate`): alone on the SM, and with the neighbours a kernel gives the issuer -- warps on tensor
    memory, warps on the arithmetic pipes, bulk copies landing in shared memory.  The kernels' clock-stamp traces are
    read against these."""
    dev = torch.device("cuda")
    cyc = torch.zeros(1, dtype=torch.int64, device=dev)
    st = torch.cuda.current_stream().cuda_stream

    def pace(code):
        for r in (8, reps, reps):                             # short warm-up launch first
            ops.check(ops.lib.saf_selftest_mma_rate(code, r, cyc.data_ptr(), ops._status_ptr(dev), st))
        ops.device_status(dev)
        return round(cyc.item() / (float(MMA_FORMS[code & 255][2]) * reps), 1)

    loads = (("alone", 0), ("tensor_memory_traffic", 512), ("arithmetic", 1024), ("bulk_copies", 2048), ("all_three", 3584))
    for form, (name, ideal, _) in enumerate(MMA_FORMS):
        row = {"op": "mma_rate", "form": name, "tensor_pipe_cycles_per_instruction": round(ideal, 1),
               "alone_zero_operands": pace(form)}
        for what, flag in loads:
            row[what] = pace(form + 256 + flag)               # random operands
        print(json.dumps(row))


def print_trace():
    """Steady-state cycle counts of one CTA's pipeline from the trace arrays of a special build."""
    import ctypes
    lib = ops.lib
    if hasattr(lib, "saf_debug_ftrace"):
        buf = (ctypes.c_longlong * (8 * 64))()
        lib.saf_debug_ftrace.argtypes = [ctypes.c_void_p]
        lib.saf_debug_ftrace(buf)
        t = [buf[e * 64:(e + 1) * 64] for e in range(8)]
        n = range(8, 40)
        mean = lambda f: sum(f(j) for j in n) / len(n)
        print(json.dumps({"trace": "flash_fwd, query tile 0 of the last row pair, cycles",
                          "period_per_key_step": (t[0][40] - t[0][8]) / 32.0,
                          "softmax_busy": mean(lambda j: t[1][j] - t[0][j]),
                          "softmax_waits_for_next_scores": mean(lambda j: t[0][j + 1] - t[1][j]),
                          "p_ready_to_issuer_saw_it": mean(lambda j: t[3][j] - t[1][j]),
                          "scores_issued_to_visible": mean(lambda j: t[0][j] - t[2][j])}))
    if hasattr(lib, "saf_debug_trace"):
        buf = (ctypes.c_longlong * (2 * 8 * 64))()
        lib.saf_debug_trace.argtypes = [ctypes.c_void_p]
        lib.saf_debug_trace(buf)
        for kern, name in ((0, "flash_bwd_dkdv, key tile 0"), (1, "flash_bwd_dq, last query tile")):
            t = [buf[(kern * 8 + e) * 64:(kern * 8 + e + 1) * 64] for e in range(8)]
            n = range(8, 40)
            mean = lambda f: sum(f(j) for j in n) / len(n)
            first = 1 if kern == 0 else 2
            print(json.dumps({"trace": name + ", cycles", "period_per_tile": (t[0][40] - t[0][8]) / 32.0,
                              "scores_visible_to_first_handover": mean(lambda j: t[first][j] - t[0][j]),
                              "dP_visible_to_dS_handed_over": mean(lambda j: t[3][j] - t[2][j]),
                              "dS_handed_over_to_next_scores_visible": mean(lambda j: t[0][j + 1] - t[3][j])}))
            if kern == 0 and t[6][8]:
                # issuer side of the dK/dV kernel: how long the 8 + 8 instructions of dV(i) and S^T(i+1) take to issue
                print(json.dumps({"trace": name + ", issuer, cycles after the scores of the tile became visible",
                                  "saw_P": mean(lambda j: t[4][j] - t[0][j]), "dV_issued": mean(lambda j: t[6][j] - t[0][j]),
                                  "next_scores_issued": mean(lambda j: t[7][j] - t[0][j]),
                                  "saw_dS": mean(lambda j: t[5][j] - t[0][j])}))
    if hasattr(lib, "saf_debug_wtrace"):
        wb = (ctypes.c_longlong * (8 * 2 * 64))()
        lib.saf_debug_wtrace.argtypes = [ctypes.c_void_p]
        lib.saf_debug_wtrace(wb)
        buf0 = (ctypes.c_longlong * (2 * 8 * 64))()
        lib.saf_debug_trace(buf0)
        n = range(8, 40)
        for evt, what in ((0, "P^T"), (1, "dS^T")):
            print(json.dumps({"trace": "flash_bwd_dkdv, %s handed over per compute warp, cycles after scores visible" % what,
                              "warps": [round(sum(wb[(w * 2 + evt) * 64 + j] - buf0[j] for j in n) / len(n)) for w in range(8)]}))


if __name__ == "__main__":
    main()
    if "--trace" in sys.argv:
        print_trace()
