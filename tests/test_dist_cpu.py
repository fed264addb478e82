"""CPU, 2 gloo ranks: the gradient bucket's segmented reduce-scatter (the one collective of the path,
src/nanochat/train/optim.cpp:425-431, 437-472) in the reference's stack layout, and what a rank does when its peer
fails before the exchange."""
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
        # in the order backward produces them: the lm_head, then the layers downwards
        order = bucket.ready_after_layer(CFG.n_layer)
        for l in reversed(range(CFG.n_layer)):
            order += bucket.ready_after_layer(l)
        assert sorted(order) == list(range(len(bucket.segments)))
        works = [bucket.reduce_scatter(i, async_op=True) for i in order]
        for w in works:
            w.wait()
        results[rank] = ({k: v.clone() for k, v in bucket.chunks.items()}, bucket.lm_chunk.clone())
    finally:
        dist.destroy_process_group()


def test_segmented_reduce_scatter_two_ranks():
    """Every rank ends up with whole matrices: entries [r * c, (r + 1) * c) of each segment of each stack, averaged
    over the ranks, in the chunk order of the reference's owned_rows (src/nanochat/train/optim.cpp:263-273, 437-472);
    the lm_head as row slices (optim.cpp:425-431)."""
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    full = []
    for rank in range(world):
        b = GradBucket(CFG, torch.device("cpu"), world)
        _fill(b, rank)
        full.append(b)
    ref = full[0]
    for name, info in ref.stack_info.items():
        avg = (full[0].stacks[name].float() + full[1].stacks[name].float()) / 2  # (K_pad, m, n)
        for rank in range(world):
            owned = ref.owned_entries(name, rank)
            assert len(owned) == info["padded"] // world
            got = results[rank][0][name].float()
            assert got.shape == (len(owned), info["m"], info["n"])
            for j, entry in enumerate(owned):  # chunk row j is the whole matrix `entry` of the stack
                # gloo sums in bf16 then divides: allow one bf16 ulp
                assert torch.allclose(got[j], avg[entry], rtol=2 ** -7, atol=1e-3), (name, rank, entry)
        # between them the ranks own every entry exactly once
        assert sorted(sum((ref.owned_entries(name, r) for r in range(world)), [])) == list(range(info["padded"]))
    avg_lm = (full[0].lm_head().float() + full[1].lm_head().float()) / 2
    rows = CFG.vocab // world
    for rank in range(world):
        assert torch.allclose(results[rank][1].float(), avg_lm[rank * rows:(rank + 1) * rows], rtol=2 ** -7, atol=1e-3)


def test_bucket_layout_is_the_reference_stack_order():
    """Stacks by shape in forward order with q, k, v adjacent (one merged weight-gradient GEMM writes them), padded to a
    multiple of the world size, at most eight segments per stack (optim.cpp:21, 222-233, 699-714)."""
    cfg = StepConfig(n_layer=24, n_embd=128, vocab=512, tokens=256, chunk_rows=128)
    C = cfg.n_embd
    for world in (1, 2, 4, 8):
        b = GradBucket(cfg, torch.device("cpu"), world)
        assert list(b.stacks) == ["muon_CxC", "muon_Cx4C", "muon_4CxC"]  # sorted by shape, as the reference's map
        assert b.stacks["muon_CxC"].shape == (96, C, C) and b.stacks["muon_4CxC"].shape == (24, 4 * C, C)
        for l in (0, 5, 23):
            qkv, o = b.matrix(l, 0), b.matrix(l, 1)
            assert qkv.shape == (3 * C, C) and qkv.is_contiguous()
            assert qkv.data_ptr() == b.stacks["muon_CxC"][4 * l].data_ptr()
            assert o.data_ptr() == b.stacks["muon_CxC"][4 * l + 3].data_ptr()
            assert b.matrix(l, 2).data_ptr() == b.stacks["muon_4CxC"][l].data_ptr()
            assert b.matrix(l, 3).data_ptr() == b.stacks["muon_Cx4C"][l].data_ptr()
        for name in b.stacks:
            segs = [s for s in b.segments if s.stack == name]
            assert len(segs) <= 8 and (world > 1 or len(segs) == 1)
            assert sum(s.count for s in segs) * world == b.stack_info[name]["padded"]
        # every segment is scheduled exactly once, none before backward has written it
        seen = []
        for l in [cfg.n_layer] + list(reversed(range(cfg.n_layer))):
            for i in b.ready_after_layer(l):
                seg = b.segments[i]
                if seg.stack != "lm_head":
                    per_layer = 4 if seg.stack == "muon_CxC" else 1
                    assert seg.first // per_layer >= l  # all its layers are at or above the one just finished
                seen.append(i)
        assert sorted(seen) == list(range(len(b.segments)))
    # a stack whose count does not divide the world size is padded with zero matrices, as the reference's K_pad
    b = GradBucket(StepConfig(n_layer=3, n_embd=128, vocab=512, tokens=256, chunk_rows=128), torch.device("cpu"), 4)
    assert b.stacks["muon_4CxC"].shape[0] == 4 and float(b.stacks["muon_4CxC"][3].abs().max()) == 0.0


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
