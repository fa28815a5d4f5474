"""One data-parallel training step of a SAF model: forward + backward under bf16 autocast, fp32 AdamW, gradients
averaged over ranks by DistributedDataParallel (NCCL over NVLink on GPUs, gloo on CPU).

Follows the reference's training loop where it touches this path: the model is wrapped as
`DDP(model, device_ids=[local_rank], broadcast_buffers=False, find_unused_parameters=True)`
(nanogpt/train.py:467-472 -- frozen layers may leave whole Q/K projections out of the graph, and the pattern
buffers never change between freeze events), one optimizer update is
`logits, loss = model(x, targets); loss.backward(); clip; optimizer.step(); optimizer.zero_grad(set_to_none=True)`
(nanogpt/bench_checkpoint_training.py:104-120), AdamW with betas (0.9, 0.95), weight decay 0.1 on matrices only
(nanogpt/model.py configure_optimizers).  The batch is sharded by sequence: rank r trains on its own micro-batch and
DDP's bucketed all-reduce, overlapped with the backward, is the only collective.

Frozen heads keep exactly-zero Q/K weight-gradient rows on every rank, so their all-reduced rows stay exactly zero
(the gradient tensors keep the canonical full size, as the reference's do).
"""
import contextlib
from types import SimpleNamespace

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel

from .workloads import WORKLOADS


def model_config(w, vocab_size=50257, n_layer=None):
    C = w["n_head"] * w["head_dim"]
    return SimpleNamespace(n_embd=C, n_head=w["n_head"], n_layer=w["n_layer"] if n_layer is None else n_layer,
                           block_size=w["T"], bias=False, dropout=0.0, position_encoding="rope",
                           rand_attn_prior_repr="dense", freeze_pattern_dtype="bfloat16", vocab_size=vocab_size,
                           rope_base=w["rope_base"])


def build_training_model(name, device, seed=1337, n_layer=None, vocab_size=50257):
    """Random-init model of a workload in fp32 (master weights), default GPT-2 init N(0, 0.02^2) from `seed` (the
    same on every rank), 25 % of the heads of every layer frozen on seeded sink+decay patterns."""
    from . import synthetic
    from .model import SafGPT
    w = WORKLOADS[name] if isinstance(name, str) else name
    cfg = model_config(w, vocab_size, n_layer)
    torch.manual_seed(seed)
    m = SafGPT(cfg)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    for li, blk in enumerate(m.transformer.h):
        fz = synthetic.frozen_heads_for_layer(w["n_head"], w["n_frozen"], seed, li)
        a, r = synthetic.sink_decay_params(len(fz), seed + 1000 + li)
        blk.main_block.freeze_heads_sink_decay(fz, a.tolist(), r.tolist())
    return m.to(device).train(), w


def param_groups(model, weight_decay):
    """Matrices decay, vectors (LayerNorm gains, biases) do not; the tied embedding appears once."""
    seen, decay, no_decay = set(), [], []
    for p in model.parameters():
        if not p.requires_grad or id(p) in seen:
            continue
        seen.add(id(p))
        (decay if p.dim() >= 2 else no_decay).append(p)
    return [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}]


class TrainStep:
    """model + optimizer + (when the process group is initialised) the DDP wrapper."""

    def __init__(self, model, lr=3e-4, weight_decay=0.1, betas=(0.9, 0.95), grad_clip=1.0, autocast_dtype=torch.bfloat16):
        self.raw = model
        dev = next(model.parameters()).device
        self.device = dev
        self.ddp = None
        if dist.is_initialized() and dist.get_world_size() > 1:
            self.ddp = DistributedDataParallel(model, device_ids=[dev.index] if dev.type == "cuda" else None,
                                               broadcast_buffers=False, find_unused_parameters=True)
        self.model = self.ddp if self.ddp is not None else model
        self.opt = torch.optim.AdamW(param_groups(model, weight_decay), lr=lr, betas=betas,
                                     fused=(dev.type == "cuda"))
        self.grad_clip = grad_clip
        self.autocast_dtype = autocast_dtype

    def forward_backward(self, idx, targets, sync=True):
        """Loss of this rank's micro-batch, gradients left in .grad (averaged over ranks when sync)."""
        ctx = contextlib.nullcontext()
        if self.ddp is not None and not sync:
            ctx = self.ddp.no_sync()
        ac = torch.autocast(device_type=self.device.type, dtype=self.autocast_dtype) \
            if self.autocast_dtype is not None else contextlib.nullcontext()
        with ctx:
            with ac:
                _, loss = self.model(idx, targets)
            loss.backward()
        return loss.detach()

    def step(self, idx, targets, sync=True):
        """One optimizer update; returns the (device) loss of this rank's micro-batch."""
        loss = self.forward_backward(idx, targets, sync=sync)
        if self.grad_clip:
            torch.nn.utils.clip_grad_norm_(self.raw.parameters(), self.grad_clip)
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss


def train_flops_per_sequence(w, vocab_size=50257):
    """Algorithmic FLOPs of forward + backward for one sequence: GEMMs 3x their forward (forward, dx, dW), live
    attention 3.5x (forward + the reference's 2.5x backward count), logits included."""
    H, hd, T, nf, L = w["n_head"], w["head_dim"], w["T"], w["n_frozen"], w["n_layer"]
    U, C = H - nf, H * hd
    gemm = 2 * T * C * ((2 * U + H) * hd + C + 8 * C) * L + 2 * T * C * vocab_size
    attn = 2 * U * T * T * hd * L
    return 3 * gemm + 3.5 * attn
