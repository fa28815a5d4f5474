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

--impl reference times that CPU restatement as the whole run (the reference project itself is Python +
Triton and cannot travel to a box without its source tree; oracle/saf_oracle.py is pinned to it by
tests/golden).
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
# DRAM bytes per launch of the mixed-attention kernel at the c2 shape (dram__bytes_read.sum + dram__bytes_write.sum
# of the ncu capture summarised in profiles/flash_fwd_hd64_c2.md); other workloads report null
ATTN_TRAFFIC_BYTES = {"c2": 279262208 + 86932736}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["bf16_tflops_sustained"], d["hbm_gbs"], "measured"
    return 1400.0, 6650.0, "fallback"


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


def cpu_reference_sample(w, steps, warmup):
    """CPU restatement of the reference's eager attention layer on the host cores: one layer of the
    workload at batch 1 and full sequence length per step; tokens/s is scaled to the full stack."""
    from oracle import saf_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    T, H, hd, nf = w["T"], w["n_head"], w["head_dim"], w["n_frozen"]
    C = H * hd
    g = torch.Generator().manual_seed(1337)
    x = torch.randn(1, T, C, generator=g)
    ws = [torch.randn(C, C, generator=g) * 0.02 for _ in range(4)]
    fz = O.frozen_heads_for_layer(H, nf, 1337, 0)
    a, r = O.sink_decay_params(nf, 2337)
    states = [1 if h in fz else 0 for h in range(H)]
    patt = O.sink_decay_pattern(a, r, T, dtype=torch.float32)      # compact (nf, T, T), addressed through pidx
    pidx = [fz.index(h) if h in fz else 0 for h in range(H)]
    rope = O.rope_cache(hd, T)
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            O.attention_layer(x, *ws, states, patt, H, rope=rope, row_chunk=2048, pidx=pidx)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
    t_layer = statistics.median(times)
    tok_s = T / (t_layer * w["n_layer"])
    sample = (f"1 of {w['n_layer']} layers, batch 1 of {w['B']}, T={T}, fp32 torch-eager restatement "
              f"(dense stored pattern for frozen heads); median of {steps} runs, x{w['n_layer']} layers")
    return tok_s, t_layer, cores, sample


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
    tok_s, t_layer, cores, sample = cpu_reference_sample(w, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": t_layer * w["n_layer"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.workload, w)},
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(key, w):
    return (f"{key}: GPT-2 124M SAF-25% attention+projection stack, {w['n_layer']} layers x "
            f"(indexed QKV GEMM + RoPE, mixed attention, c_proj), {w['n_head']} heads x {w['head_dim']}, "
            f"{w['n_frozen']} sink+decay frozen heads per layer, T={w['T']}, B={w['B']} per GPU")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scope", default="stack", choices=["stack", "block", "model"],
                    help="stack: attention+projection stack (the metric's target); block: whole transformer blocks "
                         "(LayerNorms, residuals, MLP added); model: token ids -> embedding -> blocks -> final "
                         "LayerNorm -> last-position logits")
    args = ap.parse_args()

    from saf_b200 import synthetic
    w = synthetic.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
        return

    import saf_b200
    from saf_b200 import ops, parallel
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
        run = lambda xin: model(xin)[:, 0, :]             # (B, vocab)
        result_of = lambda out: out
    else:
        layers, rope, w = synthetic.build_attention_stack(args.workload, dev, blocks=(args.scope == "block"))
        B, T, C = w["B"], w["T"], w["n_head"] * w["head_dim"]
        x_host = torch.randn(B, T, C, generator=g).bfloat16().pin_memory()
        last_host = torch.empty(B, C, dtype=torch.bfloat16).pin_memory()
        run = lambda xin: synthetic.stack_forward(layers, rope, xin)
        result_of = lambda out: out[:, -1, :]
    x_dev = x_host.to(dev, non_blocking=True)

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

        # ---- timed region 1: inputs resident in HBM ------------------------------------------
        sampler = ClockSampler(local)
        parallel.barrier()
        torch.cuda.synchronize()
        if rank == 0:
            sampler.start()
        n0 = ops.launch_count()
        ops.attention_timing(True)
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
        total_ms = ev[0].elapsed_time(ev[steps])
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
        attn0 = layers[0] if args.scope == "stack" else layers[0].main_block
        if rank != 0:
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

    ms_per_step = total_ms / steps
    value = tokens / (ms_per_step * 1e-3)
    e2e_value = tokens / (e2e_ms / steps * 1e-3)
    peak_tf, peak_hbm, peak_kind = measured_peaks()
    fl = synthetic.hot_stack_flops(w)
    live_flops_per_launch = fl["live"] / w["n_layer"] * B
    attn_mean_ms = statistics.mean(attn_ms)
    achieved = live_flops_per_launch / (attn_mean_ms * 1e-3) / 1e12
    stack_flops = (fl["live"] + fl["qkv"] + fl["oproj"] + (fl["mlp"] if args.scope != "stack" else 0)) * B
    line = {
        "metric": METRIC.replace("attention+projection stack", {"stack": "attention+projection stack", "block": "whole transformer blocks", "model": "whole model: embedding, blocks, final LayerNorm, last-position logits"}[args.scope]),
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args.workload, w) + ("; whole blocks: + LayerNorms, residuals, 4x MLP with "
                                                                   "GELU" if args.scope != "stack" else "") + ("; token ids in, last-position logits out" if args.scope == "model" else ""),
                   "l2": "per-layer working set (x 100 MB, qkv 250 MB, attention out 100 MB) exceeds the 126 MB L2",
                   "timing": "CUDA events on the launching stream, max over ranks"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                "d2h_bytes_per_step": last_host.numel() * 2},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "flash_fwd_kernel (live heads on tcgen05 + co-scheduled frozen-head scan, one launch per layer)",
                     "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                     "peak_kind": f"{peak_kind} sustained dense bf16", "traffic": ATTN_TRAFFIC_BYTES.get(args.workload),
                     "flops_per_launch": live_flops_per_launch, "ms_per_launch": attn_mean_ms,
                     "launches_timed": len(attn_ms)},
        "stack": {"tflops": stack_flops / (ms_per_step * 1e-3) / 1e12, "frac_of_peak": stack_flops / (ms_per_step * 1e-3) / 1e12 / peak_tf,
                  "attention_share_of_step": sum(attn_ms) / total_ms},
        "per_layer_ms": split,
    }
    if world == 1 and not args.no_cpu_baseline:
        tok_s, t_layer, cores, sample = cpu_reference_sample(w, 2, 1)
        line["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
