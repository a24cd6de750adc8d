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


# ---- the same on GPUs: real kernels, NCCL gather, bitwise comparison with the unsharded run

def _gpu_worker(rank, world, port, B, H, M, N, D, causal, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from triton_flashattn_b200 import flash_attention_fn

    dt = torch.bfloat16
    g = torch.Generator().manual_seed(5)  # every rank draws the same global problem
    q, k, v, do = (torch.randn(B, s, H, D, generator=g).to(dt) for s in (M, N, N, M))
    bias = (0.5 * torch.randn(B, H, M, N, generator=g)).to(dt)

    def run(qs, ks, vs, bs, dos):
        qs, ks, vs, bs = (t.contiguous().to(dev).requires_grad_() for t in (qs, ks, vs, bs))
        out = flash_attention_fn(qs, ks, vs, bs, causal, None)
        out.backward(dos.contiguous().to(dev))
        return {"out": out.detach(), "dq": qs.grad, "dk": ks.grad, "dv": vs.grad, "dbias": bs.grad}

    sh = shard_batch_heads(B, H, rank, world)
    mine = run(sh.slice_bshd(q), sh.slice_bshd(k), sh.slice_bshd(v), sh.slice_bhmn(bias), sh.slice_bshd(do))
    # the shard against the fp32 oracle, worst error over all ranks
    ref = oracle.attention_backward(sh.slice_bshd(q).to(dev), sh.slice_bshd(k).to(dev), sh.slice_bshd(v).to(dev),
                                    sh.slice_bhmn(bias).to(dev), causal, None, sh.slice_bshd(do).to(dev))
    err = torch.tensor([max((mine[n].float() - ref[n].float()).abs().max().item() for n in mine)], device=dev)
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    bad = []
    whole = run(q, k, v, bias, do) if rank == 0 else None
    for name in ("out", "dq", "dk", "dv", "dbias"):
        parts = [torch.empty_like(mine[name].contiguous()) for _ in range(world)]
        dist.all_gather(parts, mine[name].contiguous())
        if rank == 0:
            for rr, part in enumerate(parts):
                s2 = shard_batch_heads(B, H, rr, world)
                full = s2.slice_bhmn(whole[name]) if name == "dbias" else s2.slice_bshd(whole[name])
                if not torch.equal(full, part):
                    bad.append(f"{name}@rank{rr}")
    torch.cuda.synchronize()
    if rank == 0:
        out_q.put((err.item(), bad))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,causal", [(2, 4, True), (1, 4, False)])
def test_two_gpu_shards_equal_the_unsharded_gpu_result_bitwise(B, H, causal):
    """Two ranks, one GPU each, NCCL: every rank runs the CUDA kernels on its (batch, head)
    shard, out/dq/dk/dv/dbias are all_gathered and rank 0 finds them bitwise equal to its own
    unsharded run; the largest error against the fp32 oracle over all shards stays in tolerance."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, 2, port, B, H, 640, 512, 128, causal, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    err, bad = out_q.get(timeout=10)
    assert bad == [], f"shards differ from the unsharded run: {bad}"
    assert err <= 4e-2, err  # bf16 tolerance plus the 16-bit rounding of large gradients
