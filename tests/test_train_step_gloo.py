"""The data-parallel training step on CPU: two gloo ranks, each on its own micro-batch, end up with the gradients
(and, after the update, the weights) of one process training on the concatenated batch -- the property
DistributedDataParallel's gradient averaging must keep (nanogpt/train.py:467-472).  The attention modules run their
eager definition (`set_capture`), so the host logic of `saf_b200.train_step` -- seeding, DDP wrapping with
find_unused_parameters, parameter groups, the update -- is what is tested here; the CUDA kernels are not involved.
Frozen heads' Q/K weight-gradient rows are exactly zero on every rank and stay exactly zero after the all-reduce."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

TINY = dict(n_layer=2, n_head=4, head_dim=16, n_frozen=1, T=48, B=1, rope_base=10000.0)
VOCAB = 64


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _model():
    from saf_b200.train_step import build_training_model
    m, _ = build_training_model(TINY, "cpu", seed=5, vocab_size=VOCAB)
    for blk in m.transformer.h:
        blk.main_block.set_capture(True, retain_attention=False)     # eager torch path: runs on CPU
    return m


def _batch():
    g = torch.Generator().manual_seed(9)
    idx = torch.randint(0, VOCAB, (2, TINY["T"]), generator=g)
    tgt = torch.randint(0, VOCAB, (2, TINY["T"]), generator=g)
    return idx, tgt


def _worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(2)
    from saf_b200 import parallel
    from saf_b200.train_step import TrainStep
    parallel.init(backend="gloo")
    ts = TrainStep(_model(), lr=1e-2, grad_clip=0.0, autocast_dtype=None)
    assert ts.ddp is not None
    idx, tgt = _batch()
    loss = ts.forward_backward(idx[rank:rank + 1], tgt[rank:rank + 1])
    grads = {n: p.grad.numpy().copy() for n, p in ts.raw.named_parameters() if p.grad is not None}
    ts.opt.step()
    weights = {n: p.detach().numpy().copy() for n, p in ts.raw.named_parameters()}
    out.put((rank, float(loss), grads, weights))     # numpy arrays travel by value
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_match_one_process_on_the_concatenated_batch():
    from saf_b200 import synthetic
    from saf_b200.train_step import TrainStep
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=300) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # one process, both sequences
    torch.set_num_threads(2)
    ts = TrainStep(_model(), lr=1e-2, grad_clip=0.0, autocast_dtype=None)
    assert ts.ddp is None
    idx, tgt = _batch()
    loss = ts.forward_backward(idx, tgt)
    ref_g = {n: p.grad.clone() for n, p in ts.raw.named_parameters() if p.grad is not None}
    ts.opt.step()
    ref_w = {n: p.detach().clone() for n, p in ts.raw.named_parameters()}
    assert abs(0.5 * (res[0][1] + res[1][1]) - float(loss)) < 1e-5
    for rank, _, grads, weights in res:
        assert set(grads) == set(ref_g)
        for n in ref_g:
            assert torch.allclose(torch.from_numpy(grads[n]), ref_g[n], rtol=1e-4, atol=1e-6), (rank, n)
        for n in ref_w:
            assert torch.allclose(torch.from_numpy(weights[n]), ref_w[n], rtol=1e-4, atol=1e-6), (rank, n)
    # frozen heads: exactly-zero Q/K rows on both ranks after the all-reduce, live rows non-zero
    hd, H = TINY["head_dim"], TINY["n_head"]
    for li in range(TINY["n_layer"]):
        fz = synthetic.frozen_heads_for_layer(H, TINY["n_frozen"], 5, li)
        for rank, _, grads, _ in res:
            for proj in ("q_proj", "k_proj"):
                gw = torch.from_numpy(grads[f"transformer.h.{li}.main_block.{proj}.weight"])
                for h in range(H):
                    mx = gw[h * hd:(h + 1) * hd].abs().max().item()
                    assert (mx == 0.0) == (h in fz), (li, proj, h, mx)
