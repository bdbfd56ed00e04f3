"""Host-side logic of the row-sharded (tensor-parallel) path, on CPU with gloo, world size 2:
row ranges, the all-gather of output slices, and that sharded == unsharded.  The local
product is a numpy stand-in; the GPU kernels are covered by the -m gpu tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eoq_quantization_b200.tp import RowShardedLinear, gather_rows, shard_rows


class _DenseShard:
    def __init__(self, w):
        self.w = w

    def gemv(self, x):
        return x @ self.w.T


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        w = torch.randn(64, 32)
        x = torch.randn(3, 32)
        lo, hi = shard_rows(64, world, rank)
        layer = RowShardedLinear(_DenseShard(w[lo:hi]), 64)
        y = layer(x)
        ok = torch.allclose(y, x @ w.T, atol=1e-6) and y.shape == (3, 64)
        y1 = gather_rows((x[0] @ w[lo:hi].T))                        # 1-D input
        ok = ok and torch.allclose(y1, x[0] @ w.T, atol=1e-6)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_row_sharded_linear_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = sorted(q.get(timeout=5) for _ in range(2))
    assert got == [(0, True), (1, True)]


def test_shard_rows_and_single_process_gather():
    assert shard_rows(11008, 8, 3) == (4128, 5504)
    assert shard_rows(4096, 1, 0) == (0, 4096)
    with pytest.raises(ValueError):
        shard_rows(10, 4, 0)
    t = torch.arange(6.0).reshape(2, 3)
    assert gather_rows(t) is t
