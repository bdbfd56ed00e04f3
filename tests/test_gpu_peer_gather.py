"""Two-GPU parity of the fused GEMV + all-gather (peer stores over NVLink): every rank must end up with the same
full output vector as the CPU oracle computes for the unsharded layer.  One process per GPU, as in production;
skipped where fewer than two GPUs are visible."""
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int) -> None:
    import torch.distributed as dist
    from eoq_quantization_b200.fused import EOQWeight
    from eoq_quantization_b200.tp import PeerGather, shard_rows
    from oracle import oracle as O

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        n, k = 768, 1024
        rng = np.random.default_rng(5)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        codes, scales = O.quantize_absmax(w, 4, 128)
        sym = (codes + 7).astype(np.uint8)
        s16 = scales.reshape(n, k // 128).astype(np.float16)
        packed = O.pack_int4_rows(codes)
        bias = rng.standard_normal(n).astype(np.float32)
        lo, hi = shard_rows(n, world, rank)
        shard = EOQWeight.from_symbols(sym[lo:hi], s16[lo:hi])
        pg = PeerGather(slot_bytes=8 * n * 4, slots=2)
        for it in range(8):
            batch = (1, 2, 5, 8)[it % 4]
            x = np.random.default_rng(100 + it).standard_normal((batch, k)).astype(np.float32)
            ref = O.int4_linear(packed, s16.astype(np.float32).reshape(-1), n, k, 128, x, bias)
            y = pg.gemv(shard, torch.from_numpy(x).cuda(), n, slot=it & 1, bias=torch.from_numpy(bias[lo:hi]).cuda())
            got = y.cpu().numpy()                                   # synchronises: the next gather may reuse the other slot
            assert got.shape == (batch, n)
            assert O.rel_l2(got, ref) < 2e-5, (rank, it, O.rel_l2(got, ref))
        xh = torch.from_numpy(x).cuda().half()
        yh = pg.gemv(shard, xh, n, slot=0)
        refh = O.int4_linear(packed, s16.astype(np.float32).reshape(-1), n, k, 128, xh.float().cpu().numpy(), None)
        assert yh.dtype == torch.float16 and O.rel_l2(yh.float().cpu().numpy(), refh) < 1e-3
        pg.check()

        # back to back, no host synchronisation in between (slots alternate; results are copied out in stream order)
        xs = [torch.from_numpy(np.random.default_rng(200 + i).standard_normal((1, k)).astype(np.float32)).cuda() for i in range(6)]
        refs = [O.int4_linear(packed, s16.astype(np.float32).reshape(-1), n, k, 128, xi.cpu().numpy(), None) for xi in xs]
        outs = [pg.gemv(shard, xs[i % 6], n, slot=i & 1).clone() for i in range(24)]
        torch.cuda.synchronize()
        pg.check()
        for i, o in enumerate(outs):
            assert O.rel_l2(o.cpu().numpy(), refs[i % 6]) < 2e-5, (rank, i)

        # the same inside a CUDA graph, replayed
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                gouts = [pg.gemv(shard, xs[i % 6], n, slot=i & 1).clone() for i in range(8)]
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        pg.check()
        for i, o in enumerate(gouts):
            assert O.rel_l2(o.cpu().numpy(), refs[i % 6]) < 2e-5, (rank, "graph", i)
        dist.barrier()
        pg.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_gemv_all_gather_two_ranks():
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
