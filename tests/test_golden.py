"""Committed golden vectors (tests/golden/hot_path_small.npz, made by tests/golden/make_golden.py):
the CPU oracle must still reproduce them, and the CUDA path must match them without the oracle."""
import os

import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import _lib
from helpers import dev, rel_l2

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hot_path_small.npz"))
TYPES = [zb.Q4_K, zb.Q5_K, zb.Q6_K, zb.Q8_0, zb.MXFP4, zb.Q5_0, zb.Q5_1, zb.F16, zb.F32]
M, K = 9, 512


@pytest.mark.parametrize("t", TYPES, ids=[_lib.TYPE_NAMES[t] for t in TYPES])
def test_oracle_reproduces_golden(oracle, t):
    n = _lib.TYPE_NAMES[t]
    w, x = GOLD[f"{n}_w"], GOLD[f"{n}_x"]
    assert np.array_equal(oracle.dequant_rows(w, M, K, t).view(np.uint32), GOLD[f"{n}_dequant"].view(np.uint32))
    assert np.array_equal(oracle.dmmv_f64(w, t, M, K, x), GOLD[f"{n}_y"])


def test_oracle_reproduces_golden_routing_and_activation(oracle):
    logits = GOLD["route_logits"]
    for k in (1, 4, 8):
        ids, w = oracle.topk_softmax(logits, k)
        assert np.array_equal(ids, GOLD[f"route_all_k{k}_ids"]) and np.array_equal(w, GOLD[f"route_all_k{k}_w"])
        ids, w = oracle.topk_softmax_weight(logits, k)
        assert np.array_equal(ids, GOLD[f"route_topk_k{k}_ids"]) and np.array_equal(w, GOLD[f"route_topk_k{k}_w"])
    assert np.array_equal(oracle.swiglu(GOLD["act_gate"], GOLD["act_up"]), GOLD["act_swiglu"])
    assert np.array_equal(oracle.swiglu(GOLD["act_gate"], GOLD["act_up"], oai=True), GOLD["act_swiglu_oai"])


@pytest.mark.gpu
@pytest.mark.parametrize("t", TYPES, ids=[_lib.TYPE_NAMES[t] for t in TYPES])
def test_cuda_matches_golden(gpu, t):
    torch, ctx, dd = gpu
    n = _lib.TYPE_NAMES[t]
    wd, xd = dev(torch, GOLD[f"{n}_w"]), dev(torch, GOLD[f"{n}_x"])
    deq = torch.empty(M * K, dtype=torch.float32, device="cuda")
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    dd.dequantRows(t, wd, deq, 0, M, K)
    dd.recordDispatch(t, wd, xd, y, M, K)
    ctx.submit_and_wait()
    assert np.array_equal(deq.cpu().numpy().view(np.uint32), GOLD[f"{n}_dequant"].reshape(-1).view(np.uint32))
    assert rel_l2(y.cpu().numpy(), GOLD[f"{n}_y"]) <= 1e-4  # f32 accumulation against the f64 dot


@pytest.mark.gpu
def test_cuda_matches_golden_routing_and_activation(gpu):
    torch, ctx, dd = gpu
    logits = dev(torch, GOLD["route_logits"])
    for rule, key in ((zb.ROUTE_SOFTMAX_ALL_RENORM, "all"), (zb.ROUTE_TOPK_THEN_SOFTMAX, "topk")):
        for k in (1, 4, 8):
            out = torch.zeros(2 * k, dtype=torch.int32, device="cuda")
            dd.dispatchSoftmaxTopk(logits, out, 128, k, rule=rule)
            ctx.submit_and_wait()
            raw = out.cpu().numpy()
            assert np.array_equal(raw[:k].view(np.uint32), GOLD[f"route_{key}_k{k}_ids"].astype(np.uint32))
            assert np.abs(raw[k:].view(np.float32) - GOLD[f"route_{key}_k{k}_w"]).max() <= 1e-6
    g, u = dev(torch, GOLD["act_gate"]), dev(torch, GOLD["act_up"])
    for oai, key in ((False, "act_swiglu"), (True, "act_swiglu_oai")):
        y = torch.zeros(300, dtype=torch.float32, device="cuda")
        dd.dispatchSwiglu(g, u, y, 300, oai=oai)
        ctx.submit_and_wait()
        assert rel_l2(y.cpu().numpy(), GOLD[key]) <= 1e-6
