"""One process, one GPU: the training step (saf_b200/train_step.py) through the CUDA kernels -- bf16 autocast, every
GEMM of the attention path and the mixed attention forward and backward in this library, fp32 AdamW -- against the
same step on the module's eager torch path (`set_capture`, the reference's semantic definition,
nanogpt/model.py:824-844): same loss, same gradients within bf16 bars, exactly-zero Q/K rows for frozen heads, a
loss that goes down, and a clean device status word."""
import copy

import pytest
import torch

from oracle import saf_oracle as O

pytestmark = pytest.mark.gpu

SMALL = dict(n_layer=2, n_head=4, head_dim=64, n_frozen=1, T=320, B=2, rope_base=10000.0)
VOCAB = 512


def test_training_step_matches_the_eager_path_and_learns():
    from saf_b200 import ops, synthetic
    from saf_b200.train_step import TrainStep, build_training_model
    dev = torch.device("cuda")
    model, w = build_training_model(SMALL, dev, seed=3, vocab_size=VOCAB)
    eager = copy.deepcopy(model)
    for blk in eager.transformer.h:
        blk.main_block.set_capture(True, retain_attention=False)
    g = torch.Generator().manual_seed(4)
    idx = torch.randint(0, VOCAB, (w["B"], w["T"]), generator=g).to(dev)
    tgt = torch.randint(0, VOCAB, (w["B"], w["T"]), generator=g).to(dev)
    fast = TrainStep(model, lr=3e-3, grad_clip=1.0)
    slow = TrainStep(eager, lr=3e-3, grad_clip=1.0, autocast_dtype=None)     # fp32 eager
    n0 = ops.launch_count()
    l_fast = fast.forward_backward(idx, tgt)
    assert ops.launch_count() - n0 >= 2 * 14, "the training step did not run on the library"
    l_slow = slow.forward_backward(idx, tgt)
    assert abs(float(l_fast) - float(l_slow)) <= 2e-2 * float(l_slow)
    gf = dict(model.named_parameters())
    for name, p in eager.named_parameters():
        if p.grad is None:
            continue
        a = gf[name].grad
        assert a is not None, name
        assert O.rel_l2(a.float().cpu(), p.grad.float().cpu()) <= 6e-2, name
    hd, H = w["head_dim"], w["n_head"]
    for li in range(w["n_layer"]):
        fz = synthetic.frozen_heads_for_layer(H, w["n_frozen"], 3, li)
        for proj in ("q_proj", "k_proj"):
            gw = gf[f"transformer.h.{li}.main_block.{proj}.weight"].grad
            for h in range(H):
                mx = gw[h * hd:(h + 1) * hd].abs().max().item()
                assert (mx == 0.0) == (h in fz), (li, proj, h, mx)
    fast.opt.zero_grad(set_to_none=True)
    losses = [float(fast.step(idx, tgt)) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.2, losses
    assert ops.device_status(dev) == 0
