"""Device-side error reporting on a GPU, without faulting, trapping or hanging it.

A bounded wait that runs out: a two-rank communicator whose second rank is a zeroed buffer in this
process that nobody ever writes a flag into. The all-reduce kernel pushes its vector, polls its own
flag slot for the short limit the test sets, records {1, site} in the status words and returns
normally; zc_submit_and_wait turns that into ZC_ERR_TIMEOUT, the communicator refuses further
collectives, and the context keeps computing.
"""
import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import synth
from helpers import dev, out_with_canary, rel_l2

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_and_is_reported(gpu, oracle):
    torch, _, _ = gpu
    ctx = zb.Context(0, stream=torch.cuda.current_stream().cuda_stream)
    dd = zb.DmmvDispatch(ctx)
    try:
        ctx.set_wait_limit(10_000)
        ctx.comm_init(0, 2)
        silent_peer = torch.zeros(ctx.comm_buffer_bytes(), dtype=torch.uint8, device="cuda")
        ctx.comm_connect_local(1, silent_peer)
        buf = torch.full((1024,), 3.0, device="cuda")
        ctx.allreduce_sum(buf, 1024)
        with pytest.raises(zb.DeviceTimeout):
            ctx.submit_and_wait()
        assert bool((buf == 3.0).all().item()), "a timed-out all-reduce must not sum stale slots"
        with pytest.raises(zb.DeviceTimeout):      # the communicator is unusable until it is set up again
            ctx.allreduce_sum(buf, 1024)
        ctx.submit_and_wait()                       # the status words were consumed: no second report
        # the context itself still works, streaming kernels included
        g = synth.rng(8, 0)
        M, K = 256, 2048
        w = synth.quant_matrix(g, zb.Q4_K, M, K)
        x = synth.activations(g, K)
        y = out_with_canary(torch, M)
        dd.recordDispatch(zb.Q4_K, dev(torch, w), dev(torch, x), y, M, K)
        ctx.submit_and_wait()
        assert rel_l2(y[:M].cpu().numpy(), oracle.dmmv_f64(w, zb.Q4_K, M, K, x)) <= 1e-4
        # a fresh communicator on the same context works again (one rank short, so only set-up is checked)
        ctx.comm_destroy()
        ctx.comm_init(0, 2)
        ctx.comm_destroy()
    finally:
        ctx.close()


def test_two_devices_in_one_process(oracle):
    """Kernels that opt in to more than 48 KB of dynamic shared memory must do so on every device a
    process uses, not only on the first."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    g = synth.rng(9, 0)
    M, K = 512, 4096
    w = synth.quant_matrix(g, zb.Q4_K, M, K)
    w6 = synth.quant_matrix(g, zb.Q6_K, M, K)
    x = synth.activations(g, K)
    for device in (0, 1, 0):
        with torch.cuda.device(device):
            ctx = zb.Context(device, stream=torch.cuda.current_stream().cuda_stream)
            dd = zb.DmmvDispatch(ctx)
            for t, wt in ((zb.Q4_K, w), (zb.Q6_K, w6)):
                y = torch.zeros(M, device=f"cuda:{device}")
                dd.recordDispatch(t, torch.from_numpy(wt).to(f"cuda:{device}"), torch.from_numpy(x).to(f"cuda:{device}"),
                                  y, M, K)
                ctx.submit_and_wait()
                assert rel_l2(y.cpu().numpy(), oracle.dmmv_f64(wt, t, M, K, x)) <= 1e-4
            ctx.close()
