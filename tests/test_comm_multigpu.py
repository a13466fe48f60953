"""One-shot peer all-reduce (zc_allreduce_sum_f32) on two GPUs of one node: one process per GPU, IPC
handles exchanged over a gloo group, results compared with the sum formed on the host. Skipped on a
single-GPU box. No rank exits while a kernel of the other is in flight (barrier before teardown)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import zinc_b200 as zb

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ok, worst = True, 0.0
    try:
        ctx = zb.Context(rank, stream=torch.cuda.current_stream().cuda_stream)
        handles = [None] * world
        dist.all_gather_object(handles, ctx.comm_init(rank, world))
        ctx.comm_connect(handles)
        dist.barrier()
        gen = torch.Generator().manual_seed(100 + rank)
        for it in range(40):
            n = (4096, 16384, 8, 2880 + 0)[it % 4]
            host = torch.randn(n, generator=gen)
            want = host.clone()
            dist.all_reduce(want)  # two ranks: a + b is the same in either order
            buf = torch.full((n + 8,), 7.0, device="cuda")
            buf[4:4 + n] = host.cuda()
            ctx.allreduce_sum(buf, n, offset=16)
            ctx.submit_and_wait()
            got = buf.cpu()
            ok = ok and bool((got[:4] == 7.0).all()) and bool((got[4 + n:] == 7.0).all())
            worst = max(worst, float((got[4:4 + n] - want).abs().max()))
        # many back-to-back reductions without host synchronisation in between
        v = torch.ones(4096, device="cuda") * (rank + 1)
        for _ in range(10):
            ctx.allreduce_sum(v, 4096)
            v.mul_(0.5)
        ctx.submit_and_wait()
        chain = float(v[0].item())
        # all-gather, in place (each rank's slice already sits in the full vector) and out of place
        for n in (75968, 2048, 4):
            full = torch.zeros(world * n, device="cuda")
            mine = torch.arange(n, device="cuda", dtype=torch.float32) + 1000000.0 * (rank + 1)
            full[rank * n:(rank + 1) * n] = mine
            ctx.allgather(full, full, n, src_offset=rank * n * 4)
            out = torch.zeros(world * n, device="cuda")
            ctx.allgather(mine, out, n)
            ctx.submit_and_wait()
            want_full = torch.cat([torch.arange(n, dtype=torch.float32) + 1000000.0 * (r + 1) for r in range(world)])
            ok = ok and bool((full.cpu() == want_full).all()) and bool((out.cpu() == want_full).all())
        dist.barrier()
        ctx.comm_destroy()
        q.put((rank, ok, worst, chain))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gpu_allreduce():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    # v0 = r+1; each round: v = (v_0 + v_1) / 2 -> the mean 1.5 after the first round, kept afterwards
    for rank, ok, worst, chain in out:
        assert ok, "bytes outside the reduced range were touched"
        assert worst == 0.0
        assert chain == 1.5


def _worker_fused(rank: int, world: int, port: int, q):
    """A two-layer tensor-parallel decode step cut from the same seeded tensors on both ranks, the hidden-state
    sums through the exchange fused into the matvecs (rows pushed from the O / down epilogues, summed in the next
    matvec's prologue), against the unsharded step on the same GPU; eagerly and as a replayed recording."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import zinc_b200 as zb
    from zinc_b200.decode_step import DecodeStep, StepShape

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    worst = []
    side = torch.cuda.Stream()  # a recording cannot be captured on the default stream
    torch.cuda.set_stream(side)
    try:
        ctx = zb.Context(rank, stream=side.cuda_stream)
        dd = zb.DmmvDispatch(ctx)
        handles = [None] * world
        dist.all_gather_object(handles, ctx.comm_init(rank, world))
        ctx.comm_connect(handles)
        dist.barrier()

        def allgather(t, r, n):
            ctx.allgather(t, t, n, src_offset=r * n * 4)

        for shape in (StepShape(hidden=2048, n_layers=2, q_dim=2048, kv_dim=2048, ffn=4096, vocab=8192),
                      StepShape(hidden=4096, n_layers=2, q_dim=4096, kv_dim=1024, ffn=12288, vocab=4096)):
            full = DecodeStep.build(torch, dd, shape, rank=0, world=1, seed=77)
            part = DecodeStep.build(torch, dd, shape, rank=rank, world=world, seed=77, allreduce=None, allgather=allgather)
            gen = torch.Generator(device="cuda").manual_seed(4321)
            x = torch.randn(shape.hidden, device="cuda", generator=gen)
            a = torch.randn(shape.q_dim, device="cuda", generator=gen)
            f = torch.randn(shape.ffn, device="cuda", generator=gen)
            nq, nf = shape.q_dim // world, shape.ffn // world
            full.x_norm.copy_(x), full.attn_out.copy_(a), full.ffn_act_in.copy_(f)
            part.x_norm.copy_(x), part.attn_out.copy_(a[rank * nq:(rank + 1) * nq])
            part.ffn_act_in.copy_(f[rank * nf:(rank + 1) * nf])
            full.record()
            ctx.submit_and_wait()
            want_h, want_l = full.hidden.clone(), full.logits.clone()
            dist.barrier()
            part.record()
            ctx.submit_and_wait()
            for got, want in ((part.hidden, want_h), (part.logits, want_l)):
                worst.append(float(((got.double() - want.double()).norm() / want.double().norm()).item()))
            # the same as a recording replayed three times: hidden accumulates, so compare the increments
            part.hidden.zero_()
            ctx.begin_record()
            part.record()
            rec = ctx.end_record()
            dist.barrier()
            for _ in range(3):
                ctx.replay(rec)
            ctx.submit_and_wait()
            worst.append(float(((part.hidden.double() / 3 - want_h.double()).norm() / want_h.double().norm()).item()))
            ctx.free_recording(rec)
            dist.barrier()
        ctx.comm_destroy()
        q.put((rank, worst))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(240)
def test_two_gpu_fused_exchange():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_fused, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, worst in out:
        assert max(worst) <= 1e-4, (rank, worst)
