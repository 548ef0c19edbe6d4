"""Data-parallel step on real GPUs (NCCL, one process per GPU): the gradients the ranks end up with
equal those of one GPU on the whole batch, eagerly and when the step is replayed from a CUDA graph.
Skipped when fewer than two GPUs are visible."""
import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60), device_id=dev)
    from pyramid_dwconv import ConvBlock
    from pyramidconvblock_b200.parallel import GradientBucket, GraphedTrainStep, shard_batch, train_step
    torch.manual_seed(4)
    model = ConvBlock(64, kernel_size=9).to(torch.float32).to(dev)
    g = torch.Generator().manual_seed(4)
    x = torch.randn((4, 20, 24, 64), generator=g)
    go = torch.randn((4, 20, 24, 64), generator=g)
    lo, hi = shard_batch(4, rank, world)
    bucket = GradientBucket(model.parameters())
    xs = x[lo:hi].to(dev).requires_grad_(True)
    y, dx = train_step(model, bucket, xs, go[lo:hi].to(dev))
    reduced = [p.grad.clone() for p in model.parameters()]
    dx = dx.clone()
    del y        # the eager step's autograd graph must be gone before a capture (see GraphedTrainStep)
    # the same shard through the captured graph
    xg = x[lo:hi].to(dev).requires_grad_(True)
    step = GraphedTrainStep(model, bucket, xg, go[lo:hi].to(dev))
    step()
    graphed = [p.grad.clone() for p in model.parameters()]
    # one-GPU truth on the global batch (no communication: a bucket of its own is not needed)
    for p in model.parameters():
        p.grad = None
    xf = x.to(dev).requires_grad_(True)
    model(xf).backward(go.to(dev))
    ok = True
    for a, b, p in zip(reduced, graphed, model.parameters()):
        scale = float(p.grad.abs().max()) + 1e-12
        ok = ok and float((a - p.grad).abs().max()) <= 2e-5 * scale and float((b - p.grad).abs().max()) <= 2e-5 * scale
    ok = ok and float((dx - xf.grad[lo:hi]).abs().max()) <= 2e-5 * float(xf.grad.abs().max())
    ret[rank] = (bool(ok), bool(step.graphed))
    torch.cuda.synchronize(dev)
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)      # skip NCCL teardown under a live captured graph


def test_two_gpu_step_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=150)
        hung = [p for p in procs if p.is_alive()]
        for p in hung:
            p.kill()
        assert not hung, "a rank did not finish"
        assert dict(ret) == {0: (True, True), 1: (True, True)}
