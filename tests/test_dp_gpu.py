"""Data-parallel train step on two GPUs over NCCL: both ranks must end with bit-identical parameters, and those must
match a single-GPU trainer that sees the two micro-batches' averaged gradient. Skipped when fewer than two GPUs are
visible. Ranks leave only between steps; the process group gets a short timeout so a lost rank ends the test."""
import datetime
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from conftest import pkg

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _batches(cfg, steps, world):
    g = torch.Generator().manual_seed(11)
    return [[torch.randint(1, cfg.vocab, (2, cfg.seq + 1), generator=g, dtype=torch.int32) for _ in range(world)]
            for _ in range(steps)]


def _cfg():
    return pkg("gpt2").GPT2Config(vocab=512, dim=128, layers=2, heads=2, ffn=256, seq=128, dropout=0.0)


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        ptj = pkg()
        cfg = _cfg()
        t = ptj.Trainer(cfg, ptj.TrainConfig.benchmark_recipe(seed=5), device=f"cuda:{rank}", world=world, rank=rank)
        losses = []
        for ys in _batches(cfg, 3, world):
            losses.append(float(t.step(ys[rank])[0]))
        torch.cuda.synchronize()
        ret[rank] = (t.p.detach().cpu(), losses, int(ptj.operators.last_kernel_fault()))
    finally:
        dist.destroy_process_group()


def _worker_recorded(rank, world, port, ret):
    """An unrecorded and a recorded data-parallel trainer side by side in one process group (both ranks issue their
    collectives in the same order): dropout 0.1, buckets small enough to cut the recording into several graphs."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        ptj = pkg()
        cfg = pkg("gpt2").GPT2Config(vocab=512, dim=128, layers=2, heads=2, ffn=256, seq=128, dropout=0.1)
        mk = lambda graph: ptj.Trainer(cfg, ptj.TrainConfig.benchmark_recipe(seed=5, bucket_mb=0.25, cuda_graph=graph),
                                       device=f"cuda:{rank}", world=world, rank=rank)
        plain, recorded = mk(False), mk(True)
        same = True
        for ys in _batches(cfg, 6, world):
            a = plain.step(ys[rank]).clone()
            b = recorded.step(ys[rank]).clone()
            same = same and torch.equal(a, b)
        torch.cuda.synchronize()
        parts = recorded._graph[1]
        ret[rank] = (bool(same and torch.equal(plain.p, recorded.p)), len(parts), recorded.graph_replays,
                     len(recorded.reducer.buckets), int(ptj.operators.last_kernel_fault()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_recorded_graph_segments_match_unrecorded_data_parallel_steps():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker_recorded, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():
            p.kill()
            p.join(10)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank in range(world):
        same, n_parts, replays, n_buckets, fault = ret[rank]
        assert fault == 0
        assert n_buckets >= 3 and n_parts == 2 * n_buckets + 1, (n_buckets, n_parts)
        assert replays == 4, "the first two steps run unrecorded, the other four are replays"
        assert same, "recorded and unrecorded steps must agree bit for bit (losses and parameters)"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_agree_and_match_the_averaged_single_gpu_step():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:  # a rank that is still running has lost its peer or hung: end it, do not wait for it
        if p.is_alive():
            p.kill()
            p.join(10)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    (p0, l0, f0), (p1, l1, f1) = ret[0], ret[1]
    assert f0 == 0 and f1 == 0
    assert torch.equal(p0, p1), "ranks diverged"
    # single GPU, same initial weights: the two micro-batch gradients are summed by hand and the update runs with the
    # same 1/world scale the data-parallel trainer applies to its all-reduced buffer
    ptj = pkg()
    cfg = _cfg()
    tr = pkg("trainer")
    ref = ptj.Trainer(cfg, ptj.TrainConfig.benchmark_recipe(seed=5), device="cuda:0")
    ref.world = world
    for step, ys in enumerate(_batches(cfg, 3, world)):
        acc = torch.zeros_like(ref.g)
        for rank, y in enumerate(ys):
            y = y.cuda()
            seeds = tr.step_seeds(ref.tc.seed, ref.t, rank, 1 + 3 * cfg.layers)
            sorted_pos = torch.sort(y[:, :-1].reshape(-1), stable=True).indices.to(torch.int32)
            ref.engine.loss_and_grads(ref.w, ref.gv, y, True, seeds, sorted_pos=sorted_pos)
            acc += ref.g
        ref.g.copy_(acc)
        ref.apply_update(ref.tc.lr)
    torch.cuda.synchronize()
    assert torch.allclose(ref.p.cpu(), p0, rtol=1e-3, atol=1e-5), float((ref.p.cpu() - p0).abs().max())
