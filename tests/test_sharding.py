"""The multi-rank path on CPU: world_size 2 and 3 over gloo."""
import os
import socket

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

from mms_b200 import sharding


def test_shard_bounds_cover_everything_once():
    for n in (0, 1, 7, 8, 4096, 11536):
        for world in (1, 2, 3, 8):
            cuts = [sharding.shard_bounds(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1


class FakeEvaluator:
    """Scores are a fixed function of the candidate, with exact ties."""

    def get_scores(self, sols):
        return [np.float64((x * 37) % 11) / 7 for x in sols]


def _worker(rank, world, port, n, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sols = list(range(n))
        ev = sharding.ShardedEvaluator(FakeEvaluator())
        scores = ev.get_scores(sols)
        best = ev.best(sols)
        out.put((rank, [float(s) for s in scores], best))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world, n):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, out)) for r in range(world)]
    for p in procs:
        p.start()
    got = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return got


def test_two_ranks_reproduce_single_process_argmax():
    n = 45
    want = FakeEvaluator().get_scores(list(range(n)))
    for rank, scores, best in _run(2, n):
        assert scores == [float(s) for s in want]
        assert best[1] == int(np.argmax(want))           # first maximum, like np.argmax
        assert best[0] == float(np.max(want))


def test_three_ranks_with_an_empty_shard():
    n = 2                                                # rank 2 gets nothing
    want = FakeEvaluator().get_scores(list(range(n)))
    for rank, scores, best in _run(3, n):
        assert scores == [float(s) for s in want]
        assert best[1] == int(np.argmax(want))
