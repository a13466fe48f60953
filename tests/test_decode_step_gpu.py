"""The recorded decode step (config 2 shape family) against the oracle, eager and replayed."""
import numpy as np
import pytest

import zinc_b200 as zb
from helpers import rel_l2
from zinc_b200.decode_step import QWEN3_8B, DecodeStep, StepShape

pytestmark = pytest.mark.gpu


def test_qwen3_8b_bytes_per_token():
    # 36 x (Q4_K 80 216 064 + Q6_K 41 287 680) + LM head 510 504 960
    assert QWEN3_8B.layer_weight_bytes() == 121_503_744
    assert QWEN3_8B.weight_bytes() == 4_884_639_744


def test_smoke_entry():
    import __graft_entry__ as ge

    ge.smoke()


def test_recorded_step_replays_identically(gpu, oracle):
    torch, _, _ = gpu
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = zb.Context(0, stream=stream.cuda_stream)
        dd = zb.DmmvDispatch(ctx)
        shape = StepShape(hidden=512, n_layers=3, q_dim=512, kv_dim=256, ffn=1024, vocab=1031)
        step = DecodeStep.build(torch, dd, shape, seed=5)
        gen = torch.Generator(device="cuda").manual_seed(9)
        for buf in (step.x_norm, step.attn_out, step.ffn_act_in):
            buf.copy_(torch.randn(buf.shape, device="cuda", generator=gen) * 0.1)
        step.record()
        ctx.submit_and_wait()
        eager_logits = step.logits.clone()
        eager_hidden = step.hidden.clone()
        # record through the library's own capture API, replay twice
        step.hidden.zero_()
        ctx.begin_record()
        n = step.record()
        rec = ctx.end_record()
        assert n == 4 * 3 + 1  # grouped Q/K/V, O, gate+up, down per layer; LM head
        assert float(step.hidden.abs().sum()) == 0.0, "recording must not execute"
        ctx.replay(rec)
        ctx.submit_and_wait()
        assert torch.equal(step.logits, eager_logits)
        assert torch.equal(step.hidden, eager_hidden)
        ctx.replay(rec)
        ctx.submit_and_wait()
        assert rel_l2(step.hidden.cpu().numpy(), 2 * eager_hidden.cpu().numpy()) <= 1e-6
        ctx.free_recording(rec)
        want = oracle.dmmv_f64(step.head.cpu().numpy(), shape.t_head, shape.vocab, shape.hidden,
                               step.x_norm.cpu().numpy())
        assert rel_l2(step.logits.cpu().numpy(), want) <= 1e-4
