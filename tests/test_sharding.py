"""Host logic of the multi-GPU path on CPU: (batch, head) partitioning and a
world_size-2 gloo run in which every rank solves its own shard with the oracle,
the shards are gathered and the result equals the unsharded computation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import eager_oracle as oracle
from triton_flashattn_b200.sharding import shard_batch_heads


def test_shards_tile_the_grid_exactly():
    for B, H, world in ((8, 32, 1), (8, 32, 2), (8, 32, 4), (8, 32, 8), (2, 8, 4), (1, 16, 8), (4, 6, 12)):
        seen = torch.zeros(B, H, dtype=torch.int32)
        for r in range(world):
            s = shard_batch_heads(B, H, r, world)
            seen[s.b0:s.b1, s.h0:s.h1] += 1
            assert s.num_pairs == B * H // world
        assert torch.all(seen == 1)


def test_bad_partitions_are_rejected():
    with pytest.raises(ValueError):
        shard_batch_heads(3, 8, 0, 2)
    with pytest.raises(ValueError):
        shard_batch_heads(2, 3, 0, 4)
    with pytest.raises(ValueError):
        shard_batch_heads(2, 8, 5, 4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, H, M, N, D, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)  # every rank draws the same global problem
    q, k, v, do = (torch.randn(B, s, H, D, generator=g) for s in (M, N, N, M))
    bias = torch.randn(B, H, M, N, generator=g)
    sh = shard_batch_heads(B, H, rank, world)
    r = oracle.attention_backward(sh.slice_bshd(q), sh.slice_bshd(k), sh.slice_bshd(v), sh.slice_bhmn(bias),
                                  True, None, sh.slice_bshd(do))
    ok = True
    for name in ("out", "dq"):
        parts = [torch.empty_like(r[name].contiguous()) for _ in range(world)]
        dist.all_gather(parts, r[name].contiguous())
        if rank == 0:
            full = oracle.attention_backward(q, k, v, bias, True, None, do)[name]
            got = torch.empty_like(full)
            for rr, part in enumerate(parts):
                s2 = shard_batch_heads(B, H, rr, world)
                got[s2.b0:s2.b1, :, s2.h0:s2.h1] = part
            ok = ok and (got - full).abs().max().item() < 1e-5
    err = torch.tensor([0.0 if ok else 1.0])
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    if rank == 0:
        out_q.put(err.item())
    dist.destroy_process_group()


@pytest.mark.parametrize("B,H", [(2, 4), (1, 4)])
def test_two_rank_gloo_run_reproduces_the_unsharded_result(B, H):
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, B, H, 24, 40, 8, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out_q.get(timeout=10) == 0.0
