"""Multi-rank host logic on CPU: two gloo ranks shard a batch with no data-path collective and agree
on the slowest rank's time (the N>1 contract of bench.py)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, total_batch, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from saf_b200 import parallel
    r, w, _ = parallel.init(backend="gloo")
    lo, hi = parallel.batch_slice(total_batch, r, w)
    parallel.barrier()
    slow = parallel.max_over_ranks(1.0 + r)
    units = parallel.sum_over_ranks(hi - lo)
    out.put((r, lo, hi, slow, units))
    dist.destroy_process_group()


def test_two_ranks_shard_batch_and_reduce_time():
    world, total = 2, 7
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [(lo, hi) for _, lo, hi, _, _ in res] == [(0, 4), (4, 7)]
    assert all(slow == 2.0 and units == 7.0 for *_, slow, units in res)


def test_batch_slices_cover_everything():
    from saf_b200.parallel import batch_slice
    for total in (1, 4, 16, 17):
        for world in (1, 2, 4, 8):
            spans = [batch_slice(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
