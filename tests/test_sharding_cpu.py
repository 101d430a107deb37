"""CPU tests of the multi-GPU host logic: shard arithmetic, and the in-place gather run as
two gloo ranks (the data-path kernels themselves need a GPU; a torch op stands in for them
here because only the partitioning and the collective are under test)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from inductor_x_b200.sharding import OuterAxisShard, even_shard, shard_bounds


def test_shard_bounds_cover_without_overlap():
    for n in (0, 1, 7, 8, 16384, 262144 + 3):
        for world in (1, 2, 4, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)
    with pytest.raises(ValueError):
        even_shard(10, 4)
    assert even_shard(16384, 8) == 2048


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(64, 32, generator=g)  # every rank builds the same global batch

        def rowsum(chunk, out):
            torch.sum(torch.nn.functional.gelu(chunk), dim=-1, out=out)

        sh = OuterAxisShard()
        local = sh.run(rowsum, x, (), torch.float32, gather=False)
        a, b = shard_bounds(64, world, rank)
        assert torch.allclose(local, torch.nn.functional.gelu(x[a:b]).sum(-1))
        full = sh.run(rowsum, x, (), torch.float32, gather=True)
        assert torch.allclose(full, torch.nn.functional.gelu(x).sum(-1))
        # a rank that holds only its own chunk writes into its slot of the full buffer and
        # the gather fills the rest in place
        buf = torch.full((64,), float("nan"))
        sh.run_local(rowsum, x[a:b].clone(), buf, gather=False)
        assert torch.allclose(buf[a:b], torch.nn.functional.gelu(x[a:b]).sum(-1)) and bool(buf.isnan().any())
        sh.gather(buf)
        assert torch.allclose(buf, torch.nn.functional.gelu(x).sum(-1))
        ret[rank] = 1
    finally:
        dist.destroy_process_group()


def test_in_place_gather_two_gloo_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: 1, 1: 1}
