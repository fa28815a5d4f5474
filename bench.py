"""Prefill throughput of the SAF-25% attention+projection stack (GPT-2 124M shapes, 16K context).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of the hot path over one batch: for each of the 12 layers, the live-only Q/K + full
V projection (one indexed GEMM with RoPE in its epilogue), the mixed attention (tcgen05 flash for live
heads, scan for the structured frozen heads) and c_proj.  Rank r owns its own batch (weak scaling, no
data-path collective).  Prints ONE JSON line on rank 0.

  value      tokens/s over all ranks, inputs resident in HBM, device-timed (CUDA events), max over ranks
  e2e        same metric with the step's input copied from pinned host memory and the last-position
             hidden state read back, copies inside the timed region
  roofline   the dominant kernel (mixed-attention launch): algorithmic live-head FLOPs / mean launch
             duration measured with event pairs inside the timed steps, against the measured dense bf16 peak
  cpu_baseline  the CPU restatement of the reference's eager path on the host cores, bounded sample

  parity     layer 0 of the stack on one sequence of the step's own input, sampled query rows against the CPU
             oracle (computed after the timed regions)

--impl reference times that CPU restatement as the whole run: every step is the full 12-layer stack on ONE
sequence of the batch on the host cores (the reference project itself is Python + Triton and cannot travel to a
box without its source tree; oracle/saf_oracle.py is pinned to it by tests/golden).  That arm never imports the
CUDA library.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "selective-attention-freezing_b200"))

METRIC = "prefill tokens/s, SAF-25% 124M @16K ctx (attention+projection stack)"


def metric_name(key, w):
    """The headline metric for the workload it is quoted on; the same unit for the others, named for what they are."""
    if key == "c2":
        return METRIC
    if w.get("n_kv") is not None:
        return f"prefill tokens/s, SAF-25% Qwen2.5-1.5B-shaped GQA @{w['T'] // 1024}K ctx (attention+projection stack)"
    return (f"prefill tokens/s, SAF-25% {w['n_layer']} x [{w['n_head']} heads x {w['head_dim']}] @{w['T'] // 1024}K ctx "
            f"(attention+projection stack)")


def load_workloads():
    """The workload table, read by path so that the CPU reference arm does not import the package (and with it
    the CUDA library)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "saf_b200_workloads", os.path.join(ROOT, "selective-attention-freezing_b200", "saf_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.WORKLOADS


def attention_traffic_bytes(workload):
    """DRAM bytes per launch of the mixed-attention kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu
    capture), from the record the profiling step leaves beside its summary; None when there is none."""
    path = os.path.join(ROOT, "profiles", "mixed_attention_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f).get(workload)
        return None if rec is None else int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"])
    except (OSError, ValueError, KeyError):
        return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["bf16_tflops_sustained"], d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1400.0, 1590.0, 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.p = gpu_index, None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "200"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out, _ = self.p.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nme, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nme)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class CpuStack:
    """The CPU restatement of the reference's eager attention layers for one workload: per-layer weights drawn
    exactly as the CUDA arm draws them, seeded frozen-head sets, dense stored patterns for the frozen heads
    (what the reference holds for this pattern family).  One dense (n_frozen, T, T) fp32 pattern buffer is built
    once and shared by all layers (each layer addresses it through pidx; every layer reads the same number of
    pattern bytes as it would from its own), which bounds host memory at T=16384."""

    def __init__(self, w, n_layer, seed=1337):
        from oracle import saf_oracle as O
        self.O, self.w = O, w
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        T, H, hd, nf = w["T"], w["n_head"], w["head_dim"], w["n_frozen"]
        C = H * hd
        g = torch.Generator().manual_seed(seed)
        self.layers = []
        for li in range(n_layer):
            ws = [torch.randn(C, C, generator=g) * 0.02 for _ in range(4)]
            fz = O.frozen_heads_for_layer(H, nf, seed, li)
            states = [1 if h in fz else 0 for h in range(H)]
            pidx = [fz.index(h) if h in fz else 0 for h in range(H)]
            self.layers.append((ws, states, pidx))
        a, r = O.sink_decay_params(nf, seed + 1000)
        rows = torch.arange(T)
        self.patt = torch.stack([torch.cat([O.sink_decay_rows(a[i], r[i], rows[i0:i0 + 1024], T, dtype=torch.float32)
                                            for i0 in range(0, T, 1024)]) for i in range(nf)])
        self.rope = O.rope_cache(hd, T, base=w["rope_base"])
        self.x = torch.randn(1, T, C, generator=torch.Generator().manual_seed(1000))

    def step(self):
        """x -> layer_L(... layer_1(x)) on one sequence; returns seconds."""
        w = self.w
        t0 = time.perf_counter()
        h = self.x
        with torch.no_grad():
            for ws, states, pidx in self.layers:
                h = self.O.attention_layer(h, *ws, states, self.patt, w["n_head"], rope=self.rope, row_chunk=2048,
                                           pidx=pidx)
        return time.perf_counter() - t0


def cpu_reference_sample(w, steps, warmup):
    """Bounded CPU sample beside the GPU number: one layer of the workload at batch 1 and full sequence length per
    run; tokens/s is scaled to the full stack (stated in `sample`)."""
    st = CpuStack(w, 1)
    times = [st.step() for _ in range(warmup + steps)][warmup:]
    t_layer = statistics.median(times)
    tok_s = w["T"] / (t_layer * w["n_layer"])
    sample = (f"1 of {w['n_layer']} layers, batch 1 of {w['B']}, T={w['T']}, fp32 torch-eager restatement "
              f"(dense stored pattern for frozen heads); median of {steps} runs, x{w['n_layer']} layers")
    return tok_s, t_layer, st.cores, sample


class ReferenceLayerC0:
    """Benchmark configuration 0 on the reference's OWN module (nanogpt/model.py `CausalSelfAttention`, dynamic
    mode, fp32, its cheap split path on CPU tensors) -- used when a checkout of the reference is named by
    SAF_REFERENCE_ROOT; elsewhere the pinned restatement stands in."""

    def __init__(self, w, root):
        sys.path.insert(0, os.path.join(root, "nanogpt"))
        import model as M          # the reference's module; it binds its own `kernel` package (torch path on CPU)
        from oracle import saf_oracle as O
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        T, H, hd = w["T"], w["n_head"], w["head_dim"]
        C = H * hd
        cfg = M.GPTConfig(block_size=T, vocab_size=64, n_layer=1, n_head=H, n_embd=C, dropout=0.0, bias=False,
                          position_encoding="rope", rand_attn_dynamic=True, freeze_pattern_dtype="float32")
        g = torch.Generator().manual_seed(1337)
        self.attn = M.CausalSelfAttention(cfg, layer_idx=0).eval()
        with torch.no_grad():
            for lin in (self.attn.q_proj, self.attn.k_proj, self.attn.v_proj, self.attn.c_proj):
                lin.weight.copy_(torch.randn(C, C, generator=g) * 0.02)
        fz = w["frozen_heads"]
        a, r = O.sink_decay_params(len(fz), 2337)
        self.attn.freeze_heads(fz, O.sink_decay_pattern(a, r, T).float())
        self.rope = M.RotaryEmbedding(hd, T, base=w["rope_base"])(T, torch.float32)
        self.x = torch.randn(w["B"], T, C, generator=torch.Generator().manual_seed(1000))

    def step(self):
        t0 = time.perf_counter()
        with torch.no_grad():
            self.attn(self.x, rope=self.rope)
        return time.perf_counter() - t0


def run_reference(args, w):
    """CPU arm: each step is the whole stack (all layers) on one sequence of the batch.  The step count follows
    --steps but is cut so that the run ends within a few minutes; the line reports the steps actually timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget_s = float(os.environ.get("SAF_BENCH_REFERENCE_BUDGET_S", "240"))
    ref_root = os.environ.get("SAF_REFERENCE_ROOT")
    if args.workload == "c0" and ref_root and os.path.isdir(os.path.join(ref_root, "nanogpt")):
        st = ReferenceLayerC0(w, ref_root)
        t_first = st.step()
        steps = max(1, min(args.steps, int(budget_s / max(t_first, 1e-3)) - 1))
        t_step = statistics.mean([st.step() for _ in range(steps)])
        tok_s = w["B"] * w["T"] / t_step
        sample = (f"the reference's own CausalSelfAttention (cheap split path, fp32, CPU), whole batch of {w['B']} x "
                  f"{w['T']} tokens per step; {steps} timed steps after 1 warm-up step")
        print(json.dumps({
            "impl": "reference", "metric": metric_name(args.workload, w), "value": tok_s, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": t_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench_config(args.workload, w, "stack"),
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": st.cores, "kind": "reference", "sample": sample},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}), flush=True)
        return
    st = CpuStack(w, w["n_layer"])
    t_first = st.step()                                       # warm-up (page faults, thread pool)
    steps = max(1, min(args.steps, int(budget_s / max(t_first, 1e-3)) - 1))
    times = [st.step() for _ in range(steps)]
    t_step = statistics.mean(times)
    tok_s = w["T"] / t_step
    sample = (f"all {w['n_layer']} layers on 1 of {w['B']} sequences, T={w['T']}, fp32 torch-eager restatement of the "
              f"reference's attention layer (dense stored patterns for frozen heads); {steps} timed steps after 1 "
              f"warm-up step (asked for {args.steps}/{args.warmup}; cut to fit {budget_s:.0f} s)")
    line = {
        "impl": "reference", "metric": metric_name(args.workload, w), "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": 1, "ms_per_step": t_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.workload, w, "stack"),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": st.cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(key, w):
    if w.get("n_kv") is not None:
        return (f"{key}: Qwen2.5-1.5B-shaped SAF-25% grouped-query attention+projection stack, {w['n_layer']} layers x "
                f"(indexed Q(live)/K/V GEMM + RoPE base {w['rope_base']:.0e}, kvidx mixed attention, o_proj), "
                f"{w['n_head']} query / {w['n_kv']} KV heads x {w['head_dim']}, hidden {w['hidden']}, {w['n_frozen']} "
                f"sink+decay frozen query heads per layer, T={w['T']}, B={w['B']} per GPU")
    return (f"{key}: GPT-2 124M SAF-25% attention+projection stack, {w['n_layer']} layers x "
            f"(indexed QKV GEMM + RoPE, mixed attention, c_proj), {w['n_head']} heads x {w['head_dim']}, "
            f"{w['n_frozen']} sink+decay frozen heads per layer, T={w['T']}, B={w['B']} per GPU")


def bench_config(key, w, scope):
    extra = {"stack": "", "block": "; whole blocks: + LayerNorms, residuals, 4x MLP with GELU",
             "model": "; whole blocks: + LayerNorms, residuals, 4x MLP with GELU; token ids in, last-position logits out"}
    return {"workload": workload_name(key, w) + extra[scope],
            "l2": "per-layer working set (x 100 MB, qkv 250 MB, attention out 100 MB) exceeds the 126 MB L2"}


def parity_block_gqa(layer, rope, w, x_one):
    """Layer 0 of a grouped-query stack on one sequence against the CPU oracle's restatement of the reference's
    Qwen3 hybrid attention layer, 64 sampled query rows.  Runs after the timed regions."""
    from oracle import saf_oracle as O
    T, H, hd = w["T"], w["n_head"], w["head_dim"]
    with torch.inference_mode():
        y = layer(x_one, rope)
    torch.cuda.synchronize()
    rows = torch.tensor(sorted(set([0, 1, 127, 128, 255, 256, T // 2, T - 129, T - 128, T - 2, T - 1]
                                   + torch.linspace(0, T - 1, 53).long().tolist())))
    wf = {n: t.detach().float().cpu() for n, t in layer.named_parameters()}
    qrows = (torch.tensor(layer._live)[:, None] * hd + torch.arange(hd)).reshape(-1)
    x1 = x_one.float().cpu()
    has_bias = "q_proj.bias" in wf
    xb = torch.cat([x1, torch.ones(1, T, 1)], -1) if has_bias else x1

    def with_bias(wn, bn, sel=None):
        wt = wf[wn] if sel is None else wf[wn][sel]
        if not has_bias:
            return wt
        b = wf[bn] if sel is None else wf[bn][sel]
        return torch.cat([wt, b[:, None]], 1)
    torch.set_num_threads(os.cpu_count() or 1)
    oc, os_ = O.rope_cache(hd, T, base=w["rope_base"])
    with torch.no_grad():
        ref = O.gqa_attention_layer(xb, with_bias("q_proj.weight", "q_proj.bias", qrows),
                                    with_bias("k_proj.weight", "k_proj.bias"), with_bias("v_proj.weight", "v_proj.bias"),
                                    wf["o_proj.weight"], layer.frozen_mask_i32.cpu(), layer.hidx_i32.cpu(),
                                    layer.pidx_i32.cpu(), layer.kvidx_i32.cpu(), None, oc, os_, layer.scaling, rows=rows,
                                    sink_decay=(layer.sd_alpha.double().cpu(), layer.sd_rho.double().cpu()))
    got = y[:, rows.to(y.device)].float().cpu()
    return {"max_abs": O.max_abs(got, ref), "rel_l2": O.rel_l2(got, ref), "rows": int(rows.numel()),
            "against": "fp32 CPU oracle of the reference's grouped-query attention layer, layer 0, 1 sequence, all heads",
            "bar": "max_abs <= 2e-2 and rel_l2 <= 1e-2"}


def parity_block(layer, rope, w, x_one):
    """Layer 0 on one sequence of the benchmark's own input against the CPU oracle on 64 sampled query rows
    (all heads, all columns of those rows).  Runs after the timed regions."""
    from oracle import saf_oracle as O
    T, H, hd = w["T"], w["n_head"], w["head_dim"]
    with torch.inference_mode():
        y = layer(x_one, rope=rope)
    torch.cuda.synchronize()
    rows = sorted(set([0, 1, 127, 128, 255, 256, T // 2, T // 2 + 129, T - 256, T - 129, T - 128, T - 2, T - 1]
                      + torch.linspace(0, T - 1, 51).long().tolist()))
    rows = torch.tensor([r for r in rows if 0 <= r < T])
    ws = [lin.weight.detach().float().cpu() for lin in (layer.q_proj, layer.k_proj, layer.v_proj, layer.c_proj)]
    sd = layer.sd_params().double().cpu()
    torch.set_num_threads(os.cpu_count() or 1)
    with torch.no_grad():
        ref = O.attention_layer(x_one.float().cpu(), *ws, list(layer._states), None, H,
                                rope=O.rope_cache(hd, T, base=w["rope_base"]), rows=rows,
                                sink_decay=(sd[:, 0], sd[:, 1]))
    got = y[:, rows.to(y.device)].float().cpu()
    return {"max_abs": O.max_abs(got, ref), "rel_l2": O.rel_l2(got, ref), "rows": int(rows.numel()),
            "against": "fp32 CPU oracle of the reference's eager layer, layer 0, 1 sequence, all heads",
            "bar": "max_abs <= 2e-2 and rel_l2 <= 1e-2"}


def run_train(args, w):
    """One data-parallel training step per timed step: rank r trains on its own micro-batch of B sequences (weak
    scaling), gradients averaged by DDP's bucketed NCCL all-reduce overlapped with the backward, fp32 AdamW.
    `value`: token ids resident on the device; `e2e`: ids and targets copied from pinned host memory and the loss
    read back every step.  At N > 1 the same steps are timed once more without the gradient synchronisation to
    report the share of the step the all-reduce costs."""
    import saf_b200  # noqa: F401
    from saf_b200 import ops, parallel, train_step
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    rank, world, local = parallel.init()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    warmup, steps = max(args.warmup, 3), max(args.steps, 1)
    vocab = 50257
    model, w = train_step.build_training_model(args.workload, dev, n_layer=args.layers, vocab_size=vocab)
    n_layer = len(model.transformer.h)
    ts = train_step.TrainStep(model)
    B, T = w["B"], w["T"]
    g = torch.Generator().manual_seed(1000 + rank)
    ids_host = torch.randint(0, vocab, (2, B, T), generator=g, dtype=torch.int64).pin_memory()   # ids, targets
    ids_dev = ids_host.to(dev, non_blocking=True)
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def timed(fn, n):
        parallel.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        parallel.barrier()
        return parallel.max_over_ranks(e0.elapsed_time(e1), dev)

    def step_resident(sync=True):
        return ts.step(ids_dev[0], ids_dev[1], sync=sync)

    def step_e2e():
        buf = ids_host.to(dev, non_blocking=True)
        loss = ts.step(buf[0], buf[1])
        loss_host.copy_(loss.float().reshape(1), non_blocking=True)

    for _ in range(warmup):
        step_resident()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = ops.launch_count()
    ops.attention_timing(True)
    total_ms = timed(step_resident, steps)
    attn_events = ops.attention_timing(False)
    launches = ops.launch_count() - n0
    clocks = sampler.stop() if rank == 0 else None
    attn_ms = [a.elapsed_time(b) for a, b in attn_events]
    e2e_ms = timed(step_e2e, steps)
    nosync_ms = timed(lambda: step_resident(sync=False), steps) if world > 1 else None
    torch.cuda.synchronize()
    final_loss = float(loss_host.item())
    status = ops.device_status(dev)
    tokens = parallel.sum_over_ranks(B * T, dev)
    parallel.finalize()
    if rank != 0:
        return
    ms_per_step = total_ms / steps
    peak_tf, peak_burst_tf, _, peak_kind = measured_peaks()
    wl = dict(w, n_layer=n_layer)
    flops = train_step.train_flops_per_sequence(wl, vocab) * B
    live_fwd = 2.0 * B * (w["n_head"] - w["n_frozen"]) * T * T * w["head_dim"]
    attn_mean = statistics.mean(attn_ms) if attn_ms else float("nan")
    achieved = live_fwd / (attn_mean * 1e-3) / 1e12
    n_params = sum(p.numel() for p in model.parameters())
    line = {
        "metric": "training tokens/s, SAF-25% GPT (24 x [16 heads x 128], d=2048), T=8192, forward + backward + AdamW",
        "value": tokens / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: training step, {n_layer} layers x {w['n_head']} heads x {w['head_dim']}, "
                               f"{w['n_frozen']} sink+decay frozen heads per layer, MLP 4x, vocab {vocab}, T={T}, "
                               f"micro-batch {B} per GPU, bf16 autocast, fp32 AdamW, DDP (find_unused_parameters) over NCCL",
                   "l2": "activations of one layer (x 67 MB, qkv 168 MB, MLP hidden 268 MB) exceed the 126 MB L2"},
        "timing": "CUDA events on the launching stream, max over ranks",
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / steps * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": ids_host.numel() * ids_host.element_size(), "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "mixed-attention forward launch inside the training step",
                     "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                     "peak_kind": f"{peak_kind} sustained dense bf16 (kernel timed inside a long step)",
                     "frac_of_burst_peak": achieved / peak_burst_tf, "traffic": None,
                     "flops_per_launch": live_fwd, "ms_per_launch": attn_mean, "launches_timed": len(attn_ms)},
        "step": {"tflops": flops / (ms_per_step * 1e-3) / 1e12, "frac_of_peak": flops / (ms_per_step * 1e-3) / 1e12 / peak_tf,
                 "parameters": n_params, "gradient_bytes_all_reduced": 4 * n_params if world > 1 else 0,
                 "ms_per_step_without_gradient_sync": None if nosync_ms is None else nosync_ms / steps,
                 "all_reduce_share_of_step": None if nosync_ms is None else max(0.0, 1.0 - nosync_ms / total_ms),
                 "final_loss": final_loss, "device_status": status},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scope", default="stack", choices=["stack", "block", "model", "train"],
                    help="stack: attention+projection stack (the metric's target); block: whole transformer blocks "
                         "(LayerNorms, residuals, MLP added); model: token ids -> embedding -> blocks -> final "
                         "LayerNorm -> last-position logits; train: one data-parallel training step of the whole "
                         "model (forward + backward under bf16 autocast, fp32 AdamW, DDP gradient all-reduce over "
                         "NCCL), normally with --workload c3")
    ap.add_argument("--layers", type=int, default=None, help="train scope: build only this many layers (debugging)")
    args = ap.parse_args()

    w = load_workloads()[args.workload]
    if args.impl == "reference":
        run_reference(args, w)          # CPU only: the package and its CUDA library are never imported here
        return

    if args.scope == "train":
        run_train(args, w)
        return

    import saf_b200  # noqa: F401
    from saf_b200 import ops, parallel, synthetic
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    rank, world, local = parallel.init()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    g = torch.Generator().manual_seed(1000 + rank)
    if args.scope == "model":
        # the whole model: int32 token ids in, last-position logits out
        model, w = synthetic.build_model(args.workload, dev)
        layers, rope = list(model.transformer.h), None
        B, T, C = w["B"], w["T"], w["n_head"] * w["head_dim"]
        x_host = torch.randint(0, model.config.vocab_size, (B, T), generator=g, dtype=torch.int32).pin_memory()
        last_host = torch.empty(B, model.config.vocab_size, dtype=torch.bfloat16).pin_memory()
        run = lambda xin: model(xin)[0][:, 0, :]          # (B, vocab)
        result_of = lambda out: out
    elif w.get("n_kv") is not None:
        # grouped-query workload: Qwen-shaped attention modules (q_proj read for live heads only, K/V for the raw KV
        # heads, kvidx attention, o_proj) -- with --scope block the RMSNorms and the gated MLP around them
        from saf_b200 import gqa
        if args.scope == "model":
            raise SystemExit("--scope model is built for the GPT-2-shaped workloads only")
        layers, rope, w = gqa.build_gqa_stack(args.workload, dev, blocks=(args.scope == "block"))
        B, T, C = w["B"], w["T"], w["hidden"]
        x_host = torch.randn(B, T, C, generator=g).bfloat16().pin_memory()
        last_host = torch.empty(B, C, dtype=torch.bfloat16).pin_memory()
        run = lambda xin: gqa.gqa_stack_forward(layers, rope, xin)
        result_of = lambda out: out[:, -1, :]
    else:
        layers, rope, w = synthetic.build_attention_stack(args.workload, dev, blocks=(args.scope == "block"))
        B, T, C = w["B"], w["T"], w["n_head"] * w["head_dim"]
        act_dtype = getattr(torch, w.get("dtype", "bfloat16"))
        x_host = torch.randn(B, T, C, generator=g).to(act_dtype).pin_memory()
        last_host = torch.empty(B, C, dtype=act_dtype).pin_memory()
        run = lambda xin: synthetic.stack_forward(layers, rope, xin)
        result_of = lambda out: out[:, -1, :]
    x_dev = x_host.to(dev, non_blocking=True)
    small_working_set = x_host.numel() * x_host.element_size() * 3 < 126 * 2 ** 20
    l2_flush = torch.zeros(160 * 2 ** 20 // 4, dtype=torch.int32, device=dev) if small_working_set else None

    def step_resident():
        return run(x_dev)

    # end to end: every step copies its input from pinned host memory and reads its result back.  The copy
    # of step i+1 runs on a second stream into the other of two device buffers while step i computes.
    copy_stream = torch.cuda.Stream(device=dev)
    x_bufs = [torch.empty_like(x_dev), torch.empty_like(x_dev)]
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    e2e_state = {"i": 0}

    def issue_copy(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])        # the step that read this buffer has finished with it
            x_bufs[slot].copy_(x_host, non_blocking=True)
            copied[slot].record(copy_stream)

    def step_e2e():
        i = e2e_state["i"]
        slot = i & 1
        if i == 0:
            consumed[0].record()
            consumed[1].record()
            issue_copy(0)
        issue_copy(slot ^ 1)                              # next step's input, overlapped with this step
        torch.cuda.current_stream().wait_event(copied[slot])
        h = run(x_bufs[slot])
        consumed[slot].record()
        last_host.copy_(result_of(h), non_blocking=True)
        e2e_state["i"] = i + 1
        return h

    with torch.inference_mode():
        for _ in range(warmup):
            step_resident()
        torch.cuda.synchronize()
        # settle: untimed steps for about a second more, so that the timed region starts at the clocks and power
        # state of sustained load instead of the first burst after idle
        t_settle = time.perf_counter()
        while time.perf_counter() - t_settle < float(os.environ.get("SAF_BENCH_SETTLE_S", "1.0")):
            step_resident()
            torch.cuda.synchronize()

        # ---- timed region 1: inputs resident in HBM ------------------------------------------
        sampler = ClockSampler(local)
        parallel.barrier()
        torch.cuda.synchronize()
        if rank == 0:
            sampler.start()
        n0 = ops.launch_count()
        ops.attention_timing(True)
        if small_working_set:
            # the layer's tensors fit in the 126 MB L2: write a larger buffer between the timed steps (outside the
            # event pairs) so that every step starts from HBM; the step time is the sum of the pairs
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            for a_ev, b_ev in pairs:
                l2_flush.add_(1)
                a_ev.record()
                step_resident()
                b_ev.record()
        else:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
            ev[0].record()
            for i in range(steps):
                step_resident()
                ev[i + 1].record()
        torch.cuda.synchronize()
        parallel.barrier()
        attn_events = ops.attention_timing(False)
        launches = ops.launch_count() - n0
        clocks = sampler.stop() if rank == 0 else None
        total_ms = sum(a_ev.elapsed_time(b_ev) for a_ev, b_ev in pairs) if small_working_set else ev[0].elapsed_time(ev[steps])
        attn_ms = [a.elapsed_time(b) for a, b in attn_events]

        # ---- timed region 2: host buffers, copies inside ---------------------------------------
        for _ in range(2):
            step_e2e()
        torch.cuda.synchronize()
        parallel.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_e2e()
        e1.record()
        torch.cuda.synchronize()
        parallel.barrier()
        e2e_ms = e0.elapsed_time(e1)

        # per-layer split (outside the timed regions): each piece launched alone on layer 0's tensors
        is_gqa = w.get("n_kv") is not None
        attn0 = None if is_gqa else (layers[0] if args.scope == "stack" else layers[0].main_block)
        if rank != 0 or is_gqa:
            split = None
        elif args.scope == "model":
            split = synthetic.per_layer_split(attn0, model.rope(T, dev), model.transformer.wte(x_dev))
        else:
            split = synthetic.per_layer_split(attn0, rope, x_dev)

    total_ms = parallel.max_over_ranks(total_ms, dev)
    e2e_ms = parallel.max_over_ranks(e2e_ms, dev)
    tokens = parallel.sum_over_ranks(B * T, dev)
    parallel.finalize()
    if rank != 0:
        return
    parity = None
    if args.scope == "stack":
        parity = (parity_block_gqa if is_gqa else parity_block)(layers[0], rope, w, x_dev[:1])

    ms_per_step = total_ms / steps
    value = tokens / (ms_per_step * 1e-3)
    e2e_value = tokens / (e2e_ms / steps * 1e-3)
    peak_tf, peak_burst_tf, peak_hbm, peak_kind = measured_peaks()
    if is_gqa:
        from saf_b200 import gqa
        fl = gqa.gqa_stack_flops(w, blocks=(args.scope != "stack"))
    else:
        fl = synthetic.hot_stack_flops(w)
    live_flops_per_launch = fl["live"] / w["n_layer"] * B
    attn_mean_ms = statistics.mean(attn_ms)
    achieved = live_flops_per_launch / (attn_mean_ms * 1e-3) / 1e12
    stack_flops = (fl["live"] + fl["qkv"] + fl["oproj"] + (fl["mlp"] if args.scope != "stack" else 0)) * B
    line = {
        "metric": metric_name(args.workload, w).replace("attention+projection stack", {"stack": "attention+projection stack", "block": "whole transformer blocks", "model": "whole model: embedding, blocks, final LayerNorm, last-position logits"}[args.scope]),
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if w.get("dtype") == "float32" else "bf16", "data": "synthetic",
        "config": dict(bench_config(args.workload, w, args.scope), **({"l2": "working set fits the 126 MB L2: a 160 MB "
                       "buffer is rewritten between the timed steps, outside the event pairs"} if small_working_set else {})),
        "timing": "CUDA events on the launching stream, max over ranks; untimed settle period after the warm-up steps",
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                "d2h_bytes_per_step": last_host.numel() * last_host.element_size()},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "flash_fwd_persistent_kernel (live heads on tcgen05 from a tile queue + co-scheduled frozen-head scan, one launch per layer)",
                     "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                     "peak_kind": f"{peak_kind} sustained dense bf16 (kernel timed inside a long step)",
                     "frac_of_burst_peak": achieved / peak_burst_tf, "traffic": attention_traffic_bytes(args.workload),
                     "flops_per_launch": live_flops_per_launch, "ms_per_launch": attn_mean_ms,
                     "launches_timed": len(attn_ms)},
        "stack": {"tflops": stack_flops / (ms_per_step * 1e-3) / 1e12, "frac_of_peak": stack_flops / (ms_per_step * 1e-3) / 1e12 / peak_tf,
                  "attention_share_of_step": sum(attn_ms) / total_ms},
        "per_layer_ms": split,
        "parity": parity,
    }
    if world == 1 and not args.no_cpu_baseline and not is_gqa:
        tok_s, t_layer, cores, sample = cpu_reference_sample(w, 2, 1)
        line["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
