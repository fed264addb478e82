"""CPU, 2 gloo ranks: the gradient bucket's segmented reduce-scatter (the one collective of the path,
src/nanochat/train/optim.cpp:425-431, 459-468) and what a rank does when its peer fails before the exchange."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nanochat_cpp_b200.dp_step import GradBucket, StepConfig

CFG = StepConfig(n_layer=2, n_embd=128, vocab=256, tokens=256, chunk_rows=128)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fill(bucket: GradBucket, rank: int):
    g = torch.Generator().manual_seed(100 + rank)
    bucket.buffer.copy_(torch.randn(bucket.numel, generator=g).to(torch.bfloat16))


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bucket = GradBucket(CFG, torch.device("cpu"), world)
        _fill(bucket, rank)
        works = [bucket.reduce_scatter(i, async_op=True) for i in reversed(range(len(bucket.segments)))]
        for w in works:
            w.wait()
        results[rank] = [s.clone() for s in bucket.shards]
    finally:
        dist.destroy_process_group()


def test_segmented_reduce_scatter_two_ranks():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    # expectation on one process: average of the two ranks' buckets, segment by segment, rank r keeps slice r
    full = []
    for rank in range(world):
        b = GradBucket(CFG, torch.device("cpu"), 1)
        _fill(b, rank)
        full.append(b.buffer.float())
    ref = GradBucket(CFG, torch.device("cpu"), world)
    for i, (off, length) in enumerate(ref.segments):
        avg = (full[0][off:off + length] + full[1][off:off + length]) / 2
        for rank in range(world):
            want = avg[rank * length // world:(rank + 1) * length // world]
            got = results[rank][i].float()
            assert got.shape == want.shape
            # gloo sums in bf16 then divides: allow one bf16 ulp
            assert torch.allclose(got, want, rtol=2 ** -7, atol=1e-3), (i, rank)


def test_segments_must_divide_across_ranks():
    with pytest.raises(ValueError):
        GradBucket(StepConfig(n_layer=1, n_embd=128, vocab=128, tokens=128), torch.device("cpu"), world=7)


def _failing_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    bucket = GradBucket(CFG, torch.device("cpu"), world)
    _fill(bucket, rank)
    if rank == 1:
        # a rank that fails on the host between steps: it never joins the collective
        results[rank] = "left"
        os._exit(0)
    try:
        bucket.reduce_scatter(0)
        results[rank] = "completed"
    except Exception as e:  # the survivor's collective ends with an error instead of hanging
        results[rank] = f"error: {type(e).__name__}"
    os._exit(0)


def test_peer_that_never_joins_ends_the_collective_with_an_error():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    ctx = mp.spawn(_failing_worker, args=(world, _free_port(), results), nprocs=world, join=False)
    for p in ctx.processes:
        p.join(60)
        assert not p.is_alive(), "a rank hung"
    assert results[1] == "left"
    assert results[0].startswith("error"), results[0]
