"""GPU parity of the MoE expert matvecs and of the routing / activation / combine steps around them."""
import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import synth
from helpers import canary_intact, dev, out_with_canary, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-4
MOE_TYPES = [zb.Q4_K, zb.Q5_K, zb.Q6_K, zb.MXFP4, zb.Q5_1, zb.Q8_0]
IDS = [zb.TYPE_NAMES[t] for t in MOE_TYPES]


def stacked(g, t, E, M, K):
    w = synth.quant_matrix(g, t, E * M, K)
    return w, zb.expert_slice_bytes(t, M, K)


def routing_buf(ids, weights=None):
    ids = np.asarray(ids, np.uint32)
    if weights is None:
        weights = np.full(ids.size, 1.0 / ids.size, np.float32)
    return np.concatenate([ids, np.asarray(weights, np.float32).view(np.uint32)])


@pytest.mark.parametrize("t", MOE_TYPES, ids=IDS)
@pytest.mark.parametrize("shared_x", [False, True])
def test_moe_dmmv(gpu, oracle, t, shared_x):
    # recordMoeDispatch (src/compute/dmmv.zig:709-739): Y[s] = W[routing[s]] X[s*x_expert_stride..]
    torch, ctx, dd = gpu
    E, M, n_used = 5, 45, 3
    K = 512 if zb.block_size(t) == 256 else 96
    g = synth.rng(200, t)
    w, stride = stacked(g, t, E, M, K)
    ids = np.array([4, 0, 2], np.uint32)
    x = synth.activations(g, 1 if shared_x else n_used, K)
    y = out_with_canary(torch, n_used * M)
    dd.recordMoeDispatch(t, dev(torch, w), dev(torch, x), y, dev(torch, routing_buf(ids)), M, K, stride, n_used,
                         0 if shared_x else K)
    ctx.submit_and_wait()
    xs = np.repeat(x, n_used, axis=0) if shared_x else x
    want = oracle.moe_dmmv_f64(w, t, M, K, stride, ids, K, xs)
    assert canary_intact(y, n_used * M)
    assert rel_l2(y[:n_used * M].cpu().numpy(), want) <= TOL


def test_reference_fixture_q4k_moe(gpu, oracle):
    # src/compute/forward_metal.zig:11582-11681: M=65, K=512, experts {2, 0}, abs tol 0.05
    torch, ctx, dd = gpu
    w, x, ids = synth.pattern_q4k_moe()
    M, K, n_used = 65, 512, 2
    stride = zb.expert_slice_bytes(zb.Q4_K, M, K)
    y = out_with_canary(torch, n_used * M)
    dd.recordMoeDispatch(zb.Q4_K, dev(torch, w), dev(torch, x), y, dev(torch, routing_buf(ids)), M, K, stride,
                         n_used, K)
    ctx.submit_and_wait()
    got = y[:n_used * M].cpu().numpy().reshape(n_used, M)
    for s in range(n_used):
        want = oracle.dmmv_f32seq(w[int(ids[s]) * stride:(int(ids[s]) + 1) * stride], zb.Q4_K, M, K, x[s])
        assert np.max(np.abs(got[s] - want)) <= 0.05


@pytest.mark.parametrize("t", [zb.Q4_K, zb.MXFP4], ids=["q4_k", "mxfp4"])
def test_moe_fused_gate_up(gpu, oracle, t):
    torch, ctx, dd = gpu
    E, M, n_used = 4, 33, 2
    K = 512 if t == zb.Q4_K else 2880
    g = synth.rng(201, t)
    wg, stride = stacked(g, t, E, M, K)
    wu, _ = stacked(g, t, E, M, K)
    ids = np.array([3, 1], np.uint32)
    x = synth.activations(g, 1, K)
    yg, yu = out_with_canary(torch, n_used * M), out_with_canary(torch, n_used * M)
    dd.dispatchMoeFusedGateUp(t, dev(torch, wg), dev(torch, wu), dev(torch, x), yg, yu,
                              dev(torch, routing_buf(ids)), M, K, stride, n_used, 0)
    ctx.submit_and_wait()
    xs = np.repeat(x, n_used, axis=0)
    assert rel_l2(yg[:n_used * M].cpu().numpy(), oracle.moe_dmmv_f64(wg, t, M, K, stride, ids, K, xs)) <= TOL
    assert rel_l2(yu[:n_used * M].cpu().numpy(), oracle.moe_dmmv_f64(wu, t, M, K, stride, ids, K, xs)) <= TOL
    assert canary_intact(yg, n_used * M) and canary_intact(yu, n_used * M)


@pytest.mark.parametrize("t", [zb.Q4_K, zb.Q5_K, zb.Q6_K], ids=["q4_k", "q5_k", "q6_k"])
def test_moe_fused_down_acc(gpu, oracle, t):
    # hidden[r] += sum_s w_s * (W[id_s][r] . X[s])  (src/shaders/dmmv_q4k_moe_fused_down_acc.comp:74-177)
    torch, ctx, dd = gpu
    E, M, K, n_used = 6, 203, 512, 4
    g = synth.rng(202, t)
    w, stride = stacked(g, t, E, M, K)
    ids = np.array([5, 0, 3, 1], np.uint32)
    wts = np.array([0.4, 0.3, 0.2, 0.1], np.float32)
    x = synth.activations(g, n_used, K)
    h0 = synth.activations(g, M)
    y = out_with_canary(torch, M)
    y[:M] = dev(torch, h0)
    dd.dispatchMoeFusedDownAcc(t, dev(torch, w), dev(torch, x), y, dev(torch, routing_buf(ids, wts)), M, K, stride,
                               n_used, K)
    ctx.submit_and_wait()
    per = oracle.moe_dmmv_f64(w, t, M, K, stride, ids, K, x)
    want = h0 + (wts.astype(np.float64)[:, None] * per).sum(0)
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy(), want) <= TOL


def test_moe_dmmv_batched(gpu, oracle):
    # Y[t][s][M] = W[routing[t*k+s]] X[t]  (src/compute/dmmv.zig:746-792)
    torch, ctx, dd = gpu
    t = zb.Q4_K
    E, M, K, k, T = 7, 24, 512, 2, 9
    g = synth.rng(203, 0)
    w, stride = stacked(g, t, E, M, K)
    ids = g.integers(0, E, size=(T, k)).astype(np.uint32)
    X = synth.activations(g, T, K)
    Y = out_with_canary(torch, T * k * M)
    dd.recordMoeBatchedDispatch(t, dev(torch, w), dev(torch, X), Y, dev(torch, ids), M, K, stride, E, k, T, K, k * M)
    ctx.submit_and_wait()
    got = Y[:T * k * M].cpu().numpy().reshape(T, k, M)
    for tok in range(T):
        want = oracle.moe_dmmv_f64(w, t, M, K, stride, ids[tok], K, np.repeat(X[tok:tok + 1], k, axis=0))
        assert rel_l2(got[tok], want) <= TOL
    assert canary_intact(Y, T * k * M)
    with pytest.raises(zb.InvalidArgument):  # K % 256 != 0 (src/compute/dmmv.zig:767)
        dd.recordMoeBatchedDispatch(t, dev(torch, w), dev(torch, X), Y, dev(torch, ids), M, 200, stride, E, k, T, K,
                                    k * M)


TOL_TC = 5e-3  # bf16 operands on the tensor cores (prefill bar)


@pytest.mark.parametrize("t,E,M,K,k,T,pad", [
    (zb.Q4_K, 8, 192, 512, 2, 64, 0),     # 32-pair tiles, last row tile half empty
    (zb.Q4_K, 4, 256, 1024, 2, 300, 8),   # 128-pair tiles, several tiles per expert, padded token strides
    (zb.Q6_K, 8, 200, 512, 2, 64, 0),     # 420-byte rows: only 4-byte aligned
    (zb.Q6_K, 3, 128, 768, 1, 400, 0),    # 630-byte rows: only 2-byte aligned; one slot per row (down-projection form)
    (zb.MXFP4, 8, 160, 320, 2, 64, 0),    # 170-byte rows, K = 5 groups of 64: a short last block
    (zb.MXFP4, 4, 256, 2880, 2, 200, 0),  # GPT-OSS row length (1530 bytes), 128-pair tiles
    (zb.MXFP4, 16, 64, 64, 1, 40, 0),     # K = 64: one group per row, 34-byte rows
])
def test_moe_dmmv_batched_grouped(gpu, oracle, t, E, M, K, k, T, pad):
    # the same entry point with a workspace: pairs grouped by expert, tensor-core tiles
    torch, ctx, dd = gpu
    g = synth.rng(207, E * 1000 + T)
    w, stride = stacked(g, t, E, M, K)
    if stride % 16:
        pytest.skip("expert stride not 16-byte aligned: the per-pair kernel serves it")
    ids = g.integers(0, E - 1, size=(T, k)).astype(np.uint32)  # the last expert gets no pair
    ids[: T // 2, 0] = 1                                        # and expert 1 many
    xs, ys = K + pad, k * M + pad
    X = np.zeros((T, xs), np.float32)
    X[:, :K] = synth.activations(g, T, K)
    Y = out_with_canary(torch, T * ys)
    ws = torch.empty(dd.moeGroupedWorkspaceBytes(T, k, K, E), dtype=torch.uint8, device="cuda")
    dd.setWorkspace(ws)
    try:
        dd.recordMoeBatchedDispatch(t, dev(torch, w), dev(torch, X), Y, dev(torch, ids), M, K, stride, E, k, T, xs, ys)
        ctx.submit_and_wait()
    finally:
        dd.setWorkspace(None)
    got = Y[:T * ys].cpu().numpy().reshape(T, ys)
    want = np.stack([oracle.moe_dmmv_f64(w, t, M, K, stride, ids[tok], K, np.repeat(X[tok:tok + 1, :K], k, axis=0))
                     for tok in range(T)])
    have = got[:, :k * M].reshape(T, k, M)
    assert rel_l2(have, want) <= TOL_TC                                     # the bar: all outputs of the call
    assert max(rel_l2(have[tok], want[tok]) for tok in range(T)) <= 2e-2    # and no single token far off
    assert canary_intact(Y, T * ys)
    if pad:  # the padding between token rows is not written
        assert np.all(got[:, k * M:] == got[0, k * M])


@pytest.mark.parametrize("rule", [zb.ROUTE_SOFTMAX_ALL_RENORM, zb.ROUTE_TOPK_THEN_SOFTMAX])
@pytest.mark.parametrize("n,k,T", [(8, 3, 1), (256, 8, 64), (32, 4, 17), (1000, 20, 3), (2000, 6, 2), (129, 8, 5)])
def test_softmax_topk(gpu, oracle, rule, n, k, T):
    torch, ctx, dd = gpu
    g = synth.rng(204, n * 10 + rule)
    logits = synth.activations(g, T, n)
    out = torch.zeros(T * 2 * k, dtype=torch.int32, device="cuda")
    dd.dispatchSoftmaxTopk(dev(torch, logits), out, n, k, rule, T)
    ctx.submit_and_wait()
    got = out.cpu().numpy().view(np.uint32).reshape(T, 2 * k)
    fn = oracle.topk_softmax if rule == zb.ROUTE_SOFTMAX_ALL_RENORM else oracle.topk_softmax_weight
    for tok in range(T):
        ids, w = fn(logits[tok], k)
        assert np.array_equal(got[tok, :k], ids)
        assert np.max(np.abs(got[tok, k:].view(np.float32) - w)) <= 1e-6


def test_softmax_topk_reference_cases_and_bias(gpu, oracle):
    # src/compute/forward.zig:11392-11407, 11620-11710; bias add: forward.zig:6752-6754
    torch, ctx, dd = gpu

    def run(lg, k, rule, bias=None):
        out = torch.zeros(2 * k, dtype=torch.int32, device="cuda")
        dd.dispatchSoftmaxTopk(dev(torch, np.asarray(lg, np.float32)), out, len(lg), k, rule, 1,
                               bias=None if bias is None else dev(torch, np.asarray(bias, np.float32)))
        ctx.submit_and_wait()
        o = out.cpu().numpy().view(np.uint32)
        return o[:k], o[k:].view(np.float32)

    ids, w = run([1.0, 3.0, 0.5, 2.0, 4.0, 1.5, 0.1, 0.2], 3, 0)
    assert list(ids) == [4, 1, 3] and abs(w.sum() - 1) < 1e-5 and w[0] > w[1] > w[2]
    ids, w = run([1.0, 1.0, 1.0, 1.0], 2, 0)
    assert list(ids) == [0, 1] and np.allclose(w, 0.5, atol=1e-6)  # ties go to the lowest index
    ids, w = run([1.0, 1.0, 1.0, 1.0], 2, 1)
    assert list(ids) == [0, 1] and np.allclose(w, 0.5, atol=1e-6)
    ids, w = run([100.0, 0.0, -100.0], 2, 0)
    assert list(ids) == [0, 1] and w[0] > 0.99
    ids, w = run([-9.0, -2.0, -5.0], 1, 1)
    assert ids[0] == 1 and abs(w[0] - 1) < 1e-6
    lg, bias = [0.0, 0.1, 0.2, 0.3], [1.0, 0.0, 0.0, -1.0]
    ids, w = run(lg, 2, 1, bias)
    want_ids, want_w = oracle.topk_softmax_weight(np.add(lg, bias, dtype=np.float32), 2)
    assert np.array_equal(ids, want_ids) and np.allclose(w, want_w, atol=1e-6)


def test_weighted_acc_swiglu_count_pack_scatter(gpu, oracle):
    torch, ctx, dd = gpu
    g = synth.rng(205, 0)
    # moe_weighted_acc: a[i] += sum_j w_j b[j*stride+i]
    n, n_used, stride = 2048 + 3, 8, 2100
    a0 = synth.activations(g, n)
    b = synth.activations(g, n_used * stride)
    r = routing_buf(np.arange(n_used), g.uniform(0, 1, n_used).astype(np.float32))
    a = out_with_canary(torch, n)
    a[:n] = dev(torch, a0)
    dd.dispatchMoeWeightedAcc(a, dev(torch, b), dev(torch, r), n, n_used, stride)
    ctx.submit_and_wait()
    assert canary_intact(a, n)
    assert rel_l2(a[:n].cpu().numpy(), oracle.moe_weighted_acc(a0, b, r, n, n_used, stride)) <= 1e-6
    # swiglu / swiglu_oai
    gate, up = synth.activations(g, 4099) * 4, synth.activations(g, 4099) * 4
    for oai in (False, True):
        y = out_with_canary(torch, 4099)
        dd.dispatchSwiglu(dev(torch, gate), dev(torch, up), y, 4099, oai=oai)
        ctx.submit_and_wait()
        assert canary_intact(y, 4099)
        assert rel_l2(y[:4099].cpu().numpy(), oracle.swiglu(gate, up, oai=oai)) <= 1e-6
        y = out_with_canary(torch, 8192)   # a multiple of four, 16-byte aligned: the four-per-thread kernel
        g8, u8 = np.tile(gate, 2)[:8192].copy(), np.tile(up, 2)[:8192].copy()
        dd.dispatchSwiglu(dev(torch, g8), dev(torch, u8), y, 8192, oai=oai)
        ctx.submit_and_wait()
        assert canary_intact(y, 8192)
        assert rel_l2(y[:8192].cpu().numpy(), oracle.swiglu(g8, u8, oai=oai)) <= 1e-6
    # count_experts over a [tokens][layers][2k] capture buffer
    T, L, k, E, layer = 37, 3, 4, 11, 1
    cap = g.integers(0, E, size=(T, L, 2 * k)).astype(np.uint32)
    counts = torch.full((E + 4,), -1, dtype=torch.int32, device="cuda")
    dd.recordCountExperts(dev(torch, cap), counts, T, L, layer, k, E, d_offset_bytes=8)
    ctx.submit_and_wait()
    want = oracle.count_experts(cap, E, k, T, 1, 2 * k * L, layer * 2 * k)
    got = counts.cpu().numpy()
    assert np.array_equal(got[2:2 + E].astype(np.uint32), want) and got[0] == -1 and got[-1] == -1
    assert want.sum() == T * k
    with pytest.raises(zb.InvalidArgument):
        dd.recordCountExperts(dev(torch, cap), counts, T, L, L, k, E)  # layer out of range
    # route pack + scatter
    T, k, E, H = 50, 4, 16, 96
    stride = 2 * k + 2
    routing = np.zeros((T, stride), np.uint32)
    for tok in range(T):
        routing[tok, :k] = g.choice(E, size=k, replace=False)
        routing[tok, k:2 * k] = g.uniform(0, 1, k).astype(np.float32).view(np.uint32)
    cnt = torch.zeros(E, dtype=torch.int32, device="cuda")
    ids = torch.full((E * T,), -1, dtype=torch.int32, device="cuda")
    dd.dispatchMoeRoutePack(dev(torch, routing), cnt, ids, T, E, k, stride, T)
    ctx.submit_and_wait()
    wc, wi = oracle.moe_route_pack(routing, T, E, k, stride, T)
    assert np.array_equal(cnt.cpu().numpy().astype(np.uint32), wc)
    gi = ids.cpu().numpy().astype(np.uint32).reshape(E, T)
    for e in range(E):
        assert np.array_equal(gi[e, :wc[e]], wi[e, :wc[e]])
    src = synth.activations(g, T * k, H)
    dst0 = synth.activations(g, T, H)
    dst = out_with_canary(torch, T * H)
    dst[:T * H] = dev(torch, dst0.reshape(-1))
    dd.dispatchMoeRouteScatter(dev(torch, routing), dev(torch, src), dst, T, H, k, stride)
    ctx.submit_and_wait()
    want = oracle.moe_route_scatter(routing, src, dst0, T, H, k, stride)
    assert canary_intact(dst, T * H)
    assert rel_l2(dst[:T * H].cpu().numpy(), want) <= 1e-6


@pytest.mark.parametrize("M,K", [(256, 2048), (32, 2880), (7, 64)])
def test_rms_norm_dmmv_f32(gpu, oracle, M, K):
    """Fused RMS norm + f32 router matvec (src/shaders/rms_norm_dmmv_f32.comp) and the plain small-M f32
    matvec that shares its kernel."""
    torch, ctx, dd = gpu
    g = synth.rng(410, M + K)
    x = synth.activations(g, K) * np.float32(3.0)
    w = (synth.activations(g, K) * np.float32(0.1) + np.float32(1.0)).astype(np.float32)
    W = synth.activations(g, M, K) * np.float32(0.05)
    eps = 1e-6
    xn, logits = oracle.rms_norm_dmmv_f32(x, w, W, M, K, eps)
    xd, wd, Wd = dev(torch, x), dev(torch, w), dev(torch, W.reshape(-1))
    out_n = out_with_canary(torch, K)
    out_l = out_with_canary(torch, M)
    dd.dispatchRmsNormDmmvF32(xd, wd, Wd, out_n, out_l, M, K, eps)
    ctx.submit_and_wait()
    assert canary_intact(out_n, K) and canary_intact(out_l, M)
    assert rel_l2(out_n[:K].cpu().numpy(), xn) <= 1e-6
    assert rel_l2(out_l[:M].cpu().numpy(), logits) <= 1e-5
    # without the normalised-vector output, and the plain f32 matvec on the same rows
    out_l2 = out_with_canary(torch, M)
    dd.dispatchRmsNormDmmvF32(xd, wd, Wd, None, out_l2, M, K, eps)
    y = out_with_canary(torch, M)
    dd.recordDispatch(zb.F32, Wd, xd, y, M, K)
    ctx.submit_and_wait()
    assert rel_l2(out_l2[:M].cpu().numpy(), logits) <= 1e-5
    assert rel_l2(y[:M].cpu().numpy(), W.astype(np.float64) @ x.astype(np.float64)) <= 1e-5
    with pytest.raises(zb.InvalidArgument):
        dd.dispatchRmsNormDmmvF32(xd, wd, Wd, xd, out_l, M, K, eps)  # in-place normalisation races


@pytest.mark.parametrize("M,K", [(32, 2048), (5, 64)])
def test_rms_norm_dmmv_alpha_beta(gpu, oracle, M, K):
    """Fused RMS norm + the two small f32 SSM projections (src/shaders/rms_norm_dmmv_q4k_alpha_beta.comp)."""
    torch, ctx, dd = gpu
    g = synth.rng(411, M + K)
    x = synth.activations(g, K) * np.float32(2.0)
    w = (synth.activations(g, K) * np.float32(0.1) + np.float32(1.0)).astype(np.float32)
    Wa, Wb = synth.activations(g, M, K) * np.float32(0.05), synth.activations(g, M, K) * np.float32(0.05)
    xn, la = oracle.rms_norm_dmmv_f32(x, w, Wa, M, K, 1e-6)
    _, lb = oracle.rms_norm_dmmv_f32(x, w, Wb, M, K, 1e-6)
    on, oa, ob = out_with_canary(torch, K), out_with_canary(torch, M), out_with_canary(torch, M)
    dd.dispatchRmsNormDmmvAlphaBeta(dev(torch, x), dev(torch, w), dev(torch, Wa.reshape(-1)), dev(torch, Wb.reshape(-1)),
                                    on, oa, ob, M, K, 1e-6)
    ctx.submit_and_wait()
    assert canary_intact(on, K) and canary_intact(oa, M) and canary_intact(ob, M)
    assert rel_l2(on[:K].cpu().numpy(), xn) <= 1e-6
    assert rel_l2(oa[:M].cpu().numpy(), la) <= 1e-5 and rel_l2(ob[:M].cpu().numpy(), lb) <= 1e-5


@pytest.mark.parametrize("E,M,K,n_used", [(12, 512, 2048, 8), (5, 100, 1024, 3), (3, 16, 512, 2)])
def test_moe_fused_gate_up_streaming(gpu, oracle, E, M, K, n_used):
    """Shapes that take the streaming kernel with device-side expert selection (Q4_K, shared x), run
    twice in a row with different routings."""
    torch, ctx, dd = gpu
    g = synth.rng(202, E * 1000 + M)
    wg, stride = stacked(g, zb.Q4_K, E, M, K)
    wu, _ = stacked(g, zb.Q4_K, E, M, K)
    x = synth.activations(g, 1, K)
    wgd, wud, xd = dev(torch, wg), dev(torch, wu), dev(torch, x)
    xs = np.repeat(x, n_used, axis=0)
    for rep in range(2):
        ids = np.array([(5 * i + 3 * rep + 1) % E for i in range(n_used)], np.uint32)
        yg, yu = out_with_canary(torch, n_used * M), out_with_canary(torch, n_used * M)
        dd.dispatchMoeFusedGateUp(zb.Q4_K, wgd, wud, xd, yg, yu, dev(torch, routing_buf(ids)), M, K, stride, n_used, 0)
        ctx.submit_and_wait()
        assert canary_intact(yg, n_used * M) and canary_intact(yu, n_used * M)
        assert rel_l2(yg[:n_used * M].cpu().numpy(), oracle.moe_dmmv_f64(wg, zb.Q4_K, M, K, stride, ids, K, xs)) <= TOL
        assert rel_l2(yu[:n_used * M].cpu().numpy(), oracle.moe_dmmv_f64(wu, zb.Q4_K, M, K, stride, ids, K, xs)) <= TOL


@pytest.mark.parametrize("E,M,K,n_used", [(6, 300, 2880, 4), (3, 32, 512, 2)])
def test_moe_fused_gate_up_streaming_mxfp4(gpu, oracle, E, M, K, n_used):
    torch, ctx, dd = gpu
    g = synth.rng(203, E * 1000 + M)
    wg, stride = stacked(g, zb.MXFP4, E, M, K)
    wu, _ = stacked(g, zb.MXFP4, E, M, K)
    x = synth.activations(g, 1, K)
    wgd, wud, xd = dev(torch, wg), dev(torch, wu), dev(torch, x)
    xs = np.repeat(x, n_used, axis=0)
    for rep in range(2):
        ids = np.array([(5 * i + 2 * rep + E - 1) % E for i in range(n_used)], np.uint32)  # includes the last expert
        yg, yu = out_with_canary(torch, n_used * M), out_with_canary(torch, n_used * M)
        dd.dispatchMoeFusedGateUp(zb.MXFP4, wgd, wud, xd, yg, yu, dev(torch, routing_buf(ids)), M, K, stride, n_used, 0)
        ctx.submit_and_wait()
        assert canary_intact(yg, n_used * M) and canary_intact(yu, n_used * M)
        assert rel_l2(yg[:n_used * M].cpu().numpy(), oracle.moe_dmmv_f64(wg, zb.MXFP4, M, K, stride, ids, K, xs)) <= TOL
        assert rel_l2(yu[:n_used * M].cpu().numpy(), oracle.moe_dmmv_f64(wu, zb.MXFP4, M, K, stride, ids, K, xs)) <= TOL


@pytest.mark.parametrize("t,E,M,K,n_used,oai", [
    (zb.Q4_K, 12, 512, 2048, 8, False),   # streaming kernel
    (zb.Q4_K, 4, 33, 512, 2, False),      # one warp per row pair
    (zb.MXFP4, 6, 300, 2880, 4, True),    # streaming MXFP4, GPT-OSS activation
    (zb.MXFP4, 3, 32, 512, 2, True),
    (zb.Q6_K, 4, 40, 512, 2, False),
])
def test_moe_fused_gate_up_act(gpu, oracle, t, E, M, K, n_used, oai):
    # gate + up + activation in one launch = zc_moe_fused_gate_up followed by zc_swiglu / zc_swiglu_oai
    torch, ctx, dd = gpu
    g = synth.rng(209, t * 100 + M)
    wg, stride = stacked(g, t, E, M, K)
    wu, _ = stacked(g, t, E, M, K)
    x = synth.activations(g, 1, K)
    ids = np.array([(3 * i + E - 1) % E for i in range(n_used)], np.uint32)
    y = out_with_canary(torch, n_used * M)
    dd.dispatchMoeFusedGateUpAct(t, dev(torch, wg), dev(torch, wu), dev(torch, x), y, dev(torch, routing_buf(ids)),
                                 M, K, stride, n_used, 0, oai=oai)
    ctx.submit_and_wait()
    xs = np.repeat(x, n_used, axis=0)
    gate = oracle.moe_dmmv_f64(wg, t, M, K, stride, ids, K, xs).astype(np.float32).reshape(-1)
    up = oracle.moe_dmmv_f64(wu, t, M, K, stride, ids, K, xs).astype(np.float32).reshape(-1)
    want = oracle.swiglu(gate, up, oai=oai)
    assert canary_intact(y, n_used * M)
    assert rel_l2(y[:n_used * M].cpu().numpy(), want) <= TOL


@pytest.mark.parametrize("E,M,K,n_used,xs", [(6, 300, 2880, 4, 2880), (4, 64, 512, 3, 520), (3, 2880, 2880, 4, 2880)])
def test_moe_fused_down_acc_streaming_mxfp4(gpu, oracle, E, M, K, n_used, xs):
    """y += sum_s w_s W[id_s] x_s through the streaming MXFP4 kernel (slots side by side along K), with a
    padded per-slot activation stride, twice in a row."""
    torch, ctx, dd = gpu
    g = synth.rng(204, E * 1000 + M)
    w, stride = stacked(g, zb.MXFP4, E, M, K)
    wd = dev(torch, w)
    for rep in range(2):
        ids = np.array([(3 * i + rep + E - 1) % E for i in range(n_used)], np.uint32)
        wts = (g.random(n_used).astype(np.float32) + np.float32(0.1))
        x = synth.activations(g, n_used, K)
        xpad = np.zeros((n_used, xs), np.float32)
        xpad[:, :K] = x
        h0 = synth.activations(g, M)
        y = out_with_canary(torch, M)
        y[:M] = dev(torch, h0)
        dd.dispatchMoeFusedDownAcc(zb.MXFP4, wd, dev(torch, xpad.reshape(-1)), y, dev(torch, routing_buf(ids, wts)), M, K,
                                   stride, n_used, xs)
        ctx.submit_and_wait()
        per = oracle.moe_dmmv_f64(w, zb.MXFP4, M, K, stride, ids, K, x)
        want = h0 + (wts.astype(np.float64)[:, None] * per).sum(0)
        assert canary_intact(y, M)
        assert rel_l2(y[:M].cpu().numpy() - h0, want - h0) <= TOL


@pytest.mark.parametrize("E,M,K,n_used,xs", [(12, 2048, 512, 8, 512), (5, 100, 768, 3, 776), (3, 64, 2048, 2, 2048),
                                           (3, 4100, 1024, 3, 1032)])
def test_moe_fused_down_acc_streaming_q6k(gpu, oracle, E, M, K, n_used, xs):
    """y += sum_s w_s W[id_s] x_s through the streaming Q6_K kernel (rows that are not 16-byte aligned,
    slots side by side along K), twice in a row."""
    torch, ctx, dd = gpu
    g = synth.rng(205, E * 1000 + M)
    w, stride = stacked(g, zb.Q6_K, E, M, K)
    wd = dev(torch, w)
    for rep in range(2):
        ids = np.array([(3 * i + rep + E - 1) % E for i in range(n_used)], np.uint32)
        wts = (g.random(n_used).astype(np.float32) + np.float32(0.1))
        x = synth.activations(g, n_used, K)
        xpad = np.zeros((n_used, xs), np.float32)
        xpad[:, :K] = x
        h0 = synth.activations(g, M)
        y = out_with_canary(torch, M)
        y[:M] = dev(torch, h0)
        dd.dispatchMoeFusedDownAcc(zb.Q6_K, wd, dev(torch, xpad.reshape(-1)), y, dev(torch, routing_buf(ids, wts)), M, K,
                                   stride, n_used, xs)
        ctx.submit_and_wait()
        per = oracle.moe_dmmv_f64(w, zb.Q6_K, M, K, stride, ids, K, x)
        want = h0 + (wts.astype(np.float64)[:, None] * per).sum(0)
        assert canary_intact(y, M)
        assert rel_l2(y[:M].cpu().numpy() - h0, want - h0) <= TOL


@pytest.mark.parametrize("use_ws", [True, False], ids=["grouped", "per_pair"])
def test_moe_dmmv_batched_pair(gpu, oracle, use_ws):
    # gate and up in one call: equal to the two single calls on either path
    torch, ctx, dd = gpu
    t, E, M, K, k, T = zb.Q4_K, 6, 128, 512, 2, 40
    g = synth.rng(210, int(use_ws))
    wg, stride = stacked(g, t, E, M, K)
    wu, _ = stacked(g, t, E, M, K)
    ids = g.integers(0, E, size=(T, k)).astype(np.uint32)
    X = synth.activations(g, T, K)
    Yg, Yu = out_with_canary(torch, T * k * M), out_with_canary(torch, T * k * M)
    if use_ws:
        dd.setWorkspace(torch.empty(dd.moeGroupedWorkspaceBytes(T, k, K, E), dtype=torch.uint8, device="cuda"))
    try:
        n0 = ctx.launch_count
        dd.recordMoeBatchedDispatchPair(t, dev(torch, wg), dev(torch, wu), dev(torch, X), Yg, Yu, dev(torch, ids),
                                        M, K, stride, E, k, T, K, k * M)
        ctx.submit_and_wait()
        assert ctx.launch_count - n0 == (4 if use_ws else 2)   # group, gather, two tile kernels / two per-pair kernels
    finally:
        dd.setWorkspace(None)
    for Y, w in ((Yg, wg), (Yu, wu)):
        want = np.stack([oracle.moe_dmmv_f64(w, t, M, K, stride, ids[i], K, np.repeat(X[i:i + 1], k, axis=0))
                         for i in range(T)])
        assert rel_l2(Y[:T * k * M].cpu().numpy().reshape(T, k, M), want) <= (TOL_TC if use_ws else TOL)
        assert canary_intact(Y, T * k * M)


def test_moe_dmmv_batched_grouped_edges(gpu, oracle):
    # with a workspace: fewer than 16 tokens keep the f32 per-pair kernel; expert ids past n_experts are
    # skipped on both paths (their output rows stay untouched) and reported by the next submit_and_wait
    torch, ctx, dd = gpu
    t, E, M, K, k = zb.Q4_K, 4, 128, 256, 2
    g = synth.rng(208, 0)
    w, stride = stacked(g, t, E, M, K)
    ws = torch.empty(dd.moeGroupedWorkspaceBytes(64, k, K, E), dtype=torch.uint8, device="cuda")
    dd.setWorkspace(ws)
    try:
        T = 9
        ids = g.integers(0, E, size=(T, k)).astype(np.uint32)
        X = synth.activations(g, T, K)
        Y = out_with_canary(torch, T * k * M)
        dd.recordMoeBatchedDispatch(t, dev(torch, w), dev(torch, X), Y, dev(torch, ids), M, K, stride, E, k, T, K, k * M)
        ctx.submit_and_wait()
        got = Y[:T * k * M].cpu().numpy().reshape(T, k, M)
        want = np.stack([oracle.moe_dmmv_f64(w, t, M, K, stride, ids[i], K, np.repeat(X[i:i + 1], k, axis=0))
                         for i in range(T)])
        assert rel_l2(got, want) <= TOL   # f32 precision: the per-pair kernel ran

        T = 32
        ids = g.integers(0, E, size=(T, k)).astype(np.uint32)
        ids[3, 1] = E + 5      # not an expert
        ids[17, 0] = 0xFFFFFFFF
        X = synth.activations(g, T, K)
        ok = np.ones((T, k), bool)
        ok[3, 1] = ok[17, 0] = False
        safe = np.where(ok, ids, 0)
        want = np.stack([oracle.moe_dmmv_f64(w, t, M, K, stride, safe[i], K, np.repeat(X[i:i + 1], k, axis=0))
                         for i in range(T)])
        for grouped in (True, False):
            dd.setWorkspace(ws if grouped else None)
            Y = out_with_canary(torch, T * k * M, init=-7.0)
            dd.recordMoeBatchedDispatch(t, dev(torch, w), dev(torch, X), Y, dev(torch, ids), M, K, stride, E, k, T, K,
                                        k * M)
            with pytest.raises(zb.InvalidArgument):   # the bad ids are reported ...
                ctx.submit_and_wait()
            got = Y[:T * k * M].cpu().numpy().reshape(T, k, M)
            assert np.all(got[3, 1] == -7.0) and np.all(got[17, 0] == -7.0)   # ... and their rows left alone
            assert rel_l2(got[ok], want[ok]) <= (TOL_TC if grouped else TOL)
            assert canary_intact(Y, T * k * M)
    finally:
        dd.setWorkspace(None)


@pytest.mark.parametrize("cfg", ["mxfp4", "kquant_shared"])
def test_moe_decode_tensor_parallel_slices(gpu, cfg):
    # the per-rank slices of a two-rank tensor-parallel MoE step, run one after the other on this GPU
    # without the collective: the ranks' hidden vectors must add up to the single-rank result
    torch, ctx, dd = gpu
    from zinc_b200.moe_step import MoeDecode, MoeShape

    if cfg == "mxfp4":   # 5 blocks of 32: an uneven cut (96 + 64)
        shape = MoeShape(hidden=256, n_experts=8, top_k=2, ffn=160, t_gate_up=zb.MXFP4, t_down=zb.MXFP4,
                         rule=zb.ROUTE_TOPK_THEN_SOFTMAX, shared=False, oai=True, n_layers=2, biases=True)
    else:
        shape = MoeShape(hidden=512, n_experts=8, top_k=2, ffn=512, t_gate_up=zb.Q4_K, t_down=zb.Q6_K,
                         rule=zb.ROUTE_SOFTMAX_ALL_RENORM, shared=True, oai=False, n_layers=2)
    full = MoeDecode.build(torch, dd, shape, seed=5)
    n_full = full.record()
    ctx.submit_and_wait()
    want = full.hidden.cpu().numpy().astype(np.float64)
    total = np.zeros_like(want)
    for rank in range(2):
        part = MoeDecode.build(torch, dd, shape, seed=5, rank=rank, world=2, allreduce=None)
        assert part.ffn_local in ((96, 64)[rank], 256)
        n_part = part.record()
        ctx.submit_and_wait()
        total += part.hidden.cpu().numpy().astype(np.float64)
        # hidden += partial (the zeroing is a memset, not a kernel)
        assert n_part == n_full + shape.n_layers
    assert rel_l2(total, want) <= 1e-5


def test_moe_ep_filter_and_skipped_slots(gpu, oracle):
    """zc_moe_ep_filter against numpy, and every MoE kernel path with a slot that holds no expert: the slot
    reads nothing and contributes zeros (streaming Q4_K gate+up, generic paths, streaming Q6_K down)."""
    torch, ctx, dd = gpu
    g = synth.rng(211, 0)
    SKIP = 0xFFFFFFFF
    T, k = 5, 4
    ids = g.integers(0, 16, size=(T, k)).astype(np.uint32)
    wts = g.random((T, k)).astype(np.float32)
    rt = np.concatenate([ids, wts.view(np.uint32)], axis=1)
    out = torch.zeros(T * 2 * k, dtype=torch.int32, device="cuda")
    dd.dispatchMoeEpFilter(dev(torch, rt), out, k, 4, 8, n_tokens=T)
    ctx.submit_and_wait()
    got = out.cpu().numpy().view(np.uint32).reshape(T, 2 * k)
    want = np.where((ids >= 4) & (ids < 8), ids - 4, SKIP).astype(np.uint32)
    assert np.array_equal(got[:, :k], want) and np.array_equal(got[:, k:], wts.view(np.uint32))

    for E, M, K, n_used in ((12, 512, 2048, 8), (4, 33, 512, 3)):   # streaming kernel / one warp per row pair
        wg, stride = stacked(g, zb.Q4_K, E, M, K)
        wu, _ = stacked(g, zb.Q4_K, E, M, K)
        x = synth.activations(g, 1, K)
        sel = np.array([(5 * i + 1) % E for i in range(n_used)], np.uint32)
        sel[1] = SKIP
        if n_used > 4:
            sel[6] = SKIP
        yg, yu = out_with_canary(torch, n_used * M, init=5.0), out_with_canary(torch, n_used * M, init=5.0)
        dd.dispatchMoeFusedGateUp(zb.Q4_K, dev(torch, wg), dev(torch, wu), dev(torch, x), yg, yu,
                                  dev(torch, routing_buf(sel)), M, K, stride, n_used, 0)
        ctx.submit_and_wait()
        safe = np.where(sel == SKIP, 0, sel).astype(np.uint32)
        live = (sel != SKIP)
        xs = np.repeat(x, n_used, axis=0)
        for y, w in ((yg, wg), (yu, wu)):
            ref = oracle.moe_dmmv_f64(w, zb.Q4_K, M, K, stride, safe, K, xs)
            have = y[:n_used * M].cpu().numpy().reshape(n_used, M)
            assert canary_intact(y, n_used * M)
            assert np.all(have[~live] == 0.0)
            assert rel_l2(have[live], ref[live]) <= TOL

    for t, E, M, K, n_used in ((zb.Q6_K, 3, 4100, 1024, 3), (zb.Q4_K, 6, 203, 512, 4)):   # streaming Q6_K / generic
        w, stride = stacked(g, t, E, M, K)
        sel = np.array([(3 * i + E - 1) % E for i in range(n_used)], np.uint32)
        sel[1] = SKIP
        wv = (g.random(n_used).astype(np.float32) + np.float32(0.1))
        x = synth.activations(g, n_used, K)
        h0 = synth.activations(g, M)
        y = out_with_canary(torch, M)
        y[:M] = dev(torch, h0)
        dd.dispatchMoeFusedDownAcc(t, dev(torch, w), dev(torch, x.reshape(-1)), y, dev(torch, routing_buf(sel, wv)), M, K,
                                   stride, n_used, K)
        ctx.submit_and_wait()
        safe = np.where(sel == SKIP, 0, sel).astype(np.uint32)
        per = oracle.moe_dmmv_f64(w, t, M, K, stride, safe, K, x)
        wl = np.where(sel == SKIP, 0.0, wv.astype(np.float64))
        want = h0 + (wl[:, None] * per).sum(0)
        assert canary_intact(y, M)
        assert rel_l2(y[:M].cpu().numpy() - h0, want - h0) <= TOL


@pytest.mark.parametrize("world", [2, 4])
def test_moe_decode_expert_parallel_ranks(gpu, world):
    # the per-rank parts of an expert-parallel MoE step (whole experts per rank, shared expert on rank 0), run
    # one after the other on this GPU without the collective: they must add up to the single-rank result
    torch, ctx, dd = gpu
    from zinc_b200.moe_step import MoeDecode, MoeShape

    shape = MoeShape(hidden=512, n_experts=16, top_k=4, ffn=512, t_gate_up=zb.Q4_K, t_down=zb.Q6_K,
                     rule=zb.ROUTE_SOFTMAX_ALL_RENORM, shared=True, oai=False, n_layers=2)
    full = MoeDecode.build(torch, dd, shape, seed=5)
    full.record()
    ctx.submit_and_wait()
    want = full.hidden.cpu().numpy().astype(np.float64)
    total = np.zeros_like(want)
    for rank in range(world):
        part = MoeDecode.build(torch, dd, shape, seed=5, rank=rank, world=world, allreduce=None, parallel="ep")
        assert (part.e_lo, part.e_hi) == (rank * 16 // world, (rank + 1) * 16 // world) and part.ffn_local == 512
        part.record()
        ctx.submit_and_wait()
        total += part.hidden.cpu().numpy().astype(np.float64)
    assert rel_l2(total, want) <= 1e-5


@pytest.mark.parametrize("rule", [zb.ROUTE_SOFTMAX_ALL_RENORM, zb.ROUTE_TOPK_THEN_SOFTMAX])
@pytest.mark.parametrize("n,K,k,norm,bias,shared", [(256, 2048, 8, False, False, True), (32, 2880, 4, False, True, False),
                                                    (129, 4096 + 512, 8, True, True, True), (8, 64, 3, True, False, False)])
def test_moe_router_topk(gpu, oracle, rule, n, K, k, norm, bias, shared):
    """Router matvec (+ RMS norm) and expert selection in one launch, twice in a row (the arrival counter must
    come back to zero): logits against the oracle's router, the selection against the oracle's selection run on
    the logits the GPU produced, the shared slot, and the expert-parallel view of the selection."""
    torch, ctx, dd = gpu
    g = synth.rng(420, n * 7 + rule)
    W = synth.activations(g, n, K) * np.float32(0.05)
    nw = (synth.activations(g, K) * np.float32(0.1) + np.float32(1.0)).astype(np.float32)
    b = (synth.activations(g, n) * np.float32(0.5)).astype(np.float32) if bias else None
    slots = k + (1 if shared else 0)
    e_lo, e_hi = n // 4, n // 2
    Wd, nwd = dev(torch, W.reshape(-1)), dev(torch, nw)
    for rep in range(2):
        x = synth.activations(g, K) * np.float32(2.0)
        if norm:
            xn, want_logits = oracle.rms_norm_dmmv_f32(x, nw, W, n, K, 1e-6)
        else:
            xn, want_logits = x, (W.astype(np.float64) @ x.astype(np.float64)).astype(np.float32)
        lg, no = out_with_canary(torch, n), out_with_canary(torch, K)
        rt = torch.full((2 * slots + 8,), 0x7ABCDEF0, dtype=torch.int32, device="cuda")
        rl = torch.full((2 * slots + 8,), 0x7ABCDEF0, dtype=torch.int32, device="cuda")
        dd.dispatchMoeRouterTopk(dev(torch, x), Wd, lg, rt, n, K, k, rule=rule, bias=None if b is None else dev(torch, b),
                                 norm_weights=nwd if norm else None, norm_out=no if norm else None, eps=1e-6,
                                 shared_slot=shared, routing_local=rl, e_lo=e_lo, e_hi=e_hi, local_shared=(rep == 0))
        ctx.submit_and_wait()
        assert canary_intact(lg, n)
        assert bool((rt[2 * slots:] == 0x7ABCDEF0).all().item()) and bool((rl[2 * slots:] == 0x7ABCDEF0).all().item())
        got_logits = lg[:n].cpu().numpy()
        assert rel_l2(got_logits, want_logits) <= 1e-5
        if norm:
            assert canary_intact(no, K) and rel_l2(no[:K].cpu().numpy(), xn) <= 1e-6
        fn = oracle.topk_softmax if rule == zb.ROUTE_SOFTMAX_ALL_RENORM else oracle.topk_softmax_weight
        ids, w = fn(got_logits + b if b is not None else got_logits, k)
        r = rt[:2 * slots].cpu().numpy().view(np.uint32)
        assert np.array_equal(r[:k], ids)
        assert np.max(np.abs(r[slots:slots + k].view(np.float32) - w)) <= 1e-6
        if shared:
            assert r[k] == zb.SHARED_EXPERT and r[slots + k] == np.float32(1.0).view(np.uint32)
        loc = rl[:2 * slots].cpu().numpy().view(np.uint32)
        want_loc = np.where((ids >= e_lo) & (ids < e_hi), ids - e_lo, zb.SKIP_EXPERT).astype(np.uint32)
        assert np.array_equal(loc[:k], want_loc) and np.array_equal(loc[slots:], r[slots:])
        if shared:
            assert loc[k] == (zb.SHARED_EXPERT if rep == 0 else zb.SKIP_EXPERT)
    with pytest.raises(zb.InvalidArgument):
        dd.dispatchMoeRouterTopk(dev(torch, x), Wd, lg, rt, 2000, K, k)


@pytest.mark.parametrize("t,E,M,K,n_used,oai,shared,biases", [
    (zb.Q4_K, 12, 512, 2048, 8, False, True, False),    # streaming Q4_K, shared expert as the ninth slot
    (zb.Q4_K, 12, 512, 2048, 8, False, True, True),
    (zb.MXFP4, 6, 300, 2880, 4, True, False, True),     # streaming MXFP4, GPT-OSS biases and activation
    (zb.MXFP4, 6, 300, 2880, 4, True, True, True),
    (zb.Q4_K, 4, 33, 512, 2, False, True, True),        # one warp per row pair
    (zb.Q6_K, 4, 40, 512, 2, True, True, False),
])
def test_moe_gate_up_act_ex(gpu, oracle, t, E, M, K, n_used, oai, shared, biases):
    """Routed gate + up, the shared expert as one more slot, the per-expert biases and the activation in one
    launch, against the oracle's per-slot matvecs, bias adds and activation; one slot holds no expert."""
    torch, ctx, dd = gpu
    g = synth.rng(421, t * 100 + M + int(shared) + 2 * int(biases))
    wg, stride = stacked(g, t, E, M, K)
    wu, _ = stacked(g, t, E, M, K)
    sg, su = synth.quant_matrix(g, t, M, K), synth.quant_matrix(g, t, M, K)
    bg, bu = synth.activations(g, E, M), synth.activations(g, E, M)
    x = synth.activations(g, 1, K)
    ids = np.array([(3 * i + E - 1) % E for i in range(n_used)], np.uint32)
    slots = n_used + (1 if shared else 0)
    sel = np.concatenate([ids, [zb.SHARED_EXPERT]]).astype(np.uint32) if shared else ids.copy()
    sel[1] = zb.SKIP_EXPERT
    y = out_with_canary(torch, slots * M, init=3.0)
    dd.dispatchMoeGateUpActEx(t, dev(torch, wg), dev(torch, wu), dev(torch, x), y, dev(torch, routing_buf(sel)), M, K, stride,
                              slots, shared=(dev(torch, sg), dev(torch, su)) if shared else None,
                              biases=(dev(torch, bg.reshape(-1)), dev(torch, bu.reshape(-1))) if biases else None, oai=oai)
    ctx.submit_and_wait()
    xs = np.repeat(x, n_used, axis=0)
    gate = oracle.moe_dmmv_f64(wg, t, M, K, stride, ids, K, xs).astype(np.float32)
    up = oracle.moe_dmmv_f64(wu, t, M, K, stride, ids, K, xs).astype(np.float32)
    if biases:
        gate, up = gate + bg[ids], up + bu[ids]
    if shared:
        gate = np.concatenate([gate, oracle.dmmv_f64(sg, t, M, K, x[0]).astype(np.float32)[None]])
        up = np.concatenate([up, oracle.dmmv_f64(su, t, M, K, x[0]).astype(np.float32)[None]])
    want = oracle.swiglu(gate.reshape(-1), up.reshape(-1), oai=oai).reshape(slots, M)
    have = y[:slots * M].cpu().numpy().reshape(slots, M)
    live = np.ones(slots, bool)
    live[1] = False
    assert canary_intact(y, slots * M)
    assert np.all(have[1] == 0.0)
    assert rel_l2(have[live], want[live]) <= TOL


@pytest.mark.parametrize("t,E,M,K,n_used,shared,bias", [
    (zb.Q6_K, 12, 2048, 512, 8, True, False),    # streaming Q6_K, shared expert as the ninth slot
    (zb.Q6_K, 5, 2100, 768, 3, True, True),      # rows that are not 16-byte aligned
    (zb.MXFP4, 6, 2880, 2880, 4, False, True),   # streaming MXFP4 with the down bias
    (zb.MXFP4, 3, 300, 2880, 3, True, True),
    (zb.Q4_K, 6, 203, 512, 4, True, True),       # generic kernel
])
def test_moe_down_acc_ex(gpu, oracle, t, E, M, K, n_used, shared, bias):
    """y += sum_s w_s (W[id_s] x_s + bias[id_s]) with the shared expert as one more slot (its own matrix, no
    bias), against the oracle; one slot holds no expert."""
    torch, ctx, dd = gpu
    g = synth.rng(422, t * 100 + M + int(shared) + 2 * int(bias))
    w, stride = stacked(g, t, E, M, K)
    sd = synth.quant_matrix(g, t, M, K)
    bd = synth.activations(g, E, M)
    slots = n_used + (1 if shared else 0)
    ids = np.array([(3 * i + E - 1) % E for i in range(n_used)], np.uint32)
    sel = np.concatenate([ids, [zb.SHARED_EXPERT]]).astype(np.uint32) if shared else ids.copy()
    sel[1] = zb.SKIP_EXPERT
    wts = (g.random(slots).astype(np.float32) + np.float32(0.1))
    x = synth.activations(g, slots, K)
    h0 = synth.activations(g, M)
    y = out_with_canary(torch, M)
    y[:M] = dev(torch, h0)
    dd.dispatchMoeDownAccEx(t, dev(torch, w), dev(torch, x.reshape(-1)), y, dev(torch, routing_buf(sel, wts)), M, K, stride,
                            slots, K, shared=dev(torch, sd) if shared else None,
                            bias=dev(torch, bd.reshape(-1)) if bias else None)
    ctx.submit_and_wait()
    per = oracle.moe_dmmv_f64(w, t, M, K, stride, ids, K, x[:n_used])
    if bias:
        per = per + bd[ids].astype(np.float64)
    if shared:
        per = np.concatenate([per, oracle.dmmv_f64(sd, t, M, K, x[n_used])[None]])
    wl = wts.astype(np.float64).copy()
    wl[1] = 0.0
    want = h0 + (wl[:, None] * per).sum(0)
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy() - h0, want - h0) <= TOL


def test_moe_decode_fused_equals_dispatch_sequence(gpu):
    """The three-launch layer (router + selection, gate + up + activation, down + sum) against the one launch per
    dispatch sequence on the same weights: a Qwen-shaped layer with a shared expert and a GPT-OSS-shaped one with
    biases."""
    torch, ctx, dd = gpu
    from zinc_b200.moe_step import MoeDecode, MoeShape
    shapes = (MoeShape(hidden=2048, n_experts=32, top_k=8, ffn=512, t_gate_up=zb.Q4_K, t_down=zb.Q6_K,
                       rule=zb.ROUTE_SOFTMAX_ALL_RENORM, shared=True, oai=False, n_layers=2),
              MoeShape(hidden=2880, n_experts=8, top_k=4, ffn=2880, t_gate_up=zb.MXFP4, t_down=zb.MXFP4,
                       rule=zb.ROUTE_TOPK_THEN_SOFTMAX, shared=False, oai=True, n_layers=2, biases=True))
    for shape in shapes:
        a = MoeDecode.build(torch, dd, shape, seed=9, fused=False)
        b = MoeDecode.build(torch, dd, shape, seed=9, fused=True)
        na, nb = a.record(), b.record()
        ctx.submit_and_wait()
        assert nb == 3 * shape.n_layers and na > nb
        ha, hb = a.hidden.double(), b.hidden.double()
        assert float(((ha - hb).norm() / ha.norm()).item()) <= 1e-5


@pytest.mark.parametrize("world", [2, 4])
def test_moe_prefill_expert_parallel_ranks(gpu, world):
    """The per-rank parts of an expert-parallel MoE prefill layer (whole experts per rank, routing filtered to
    them, absent pairs neither grouped nor summed), run one after the other on this GPU, add up to the layer on
    one rank; and zc_moe_ep_filter's ids-only rows against numpy."""
    torch, ctx, dd = gpu
    from zinc_b200.moe_step import MoePrefill, MoeShape
    shape = MoeShape(hidden=512, n_experts=16, top_k=4, ffn=512, t_gate_up=zb.Q4_K, t_down=zb.Q6_K,
                     rule=zb.ROUTE_SOFTMAX_ALL_RENORM, shared=False, oai=False, n_layers=1)
    T = 96
    full = MoePrefill.build(torch, dd, shape, T, seed=13)
    dd.setWorkspace(full.workspace)
    try:
        full.record()
        ctx.submit_and_wait()
        want = full.hidden.double().cpu()
        total = torch.zeros_like(want)
        ids = full.routing.view(T, 2 * shape.top_k)[:, :shape.top_k].cpu().numpy().view(np.uint32)
        for rank in range(world):
            part = MoePrefill.build(torch, dd, shape, T, seed=13, rank=rank, world=world)
            assert torch.equal(part.routing, full.routing) and torch.equal(part.X, full.X)
            dd.setWorkspace(part.workspace)
            part.record()
            ctx.submit_and_wait()
            total += part.hidden.double().cpu()
            lo, hi = part.e_lo, part.e_hi
            want_ids = np.where((ids >= lo) & (ids < hi), ids - lo, zb.SKIP_EXPERT).astype(np.uint32)
            assert np.array_equal(part.ids_local.cpu().numpy().view(np.uint32).reshape(T, -1), want_ids)
            assert np.array_equal(part.routing_local.view(T, -1)[:, :shape.top_k].cpu().numpy().view(np.uint32), want_ids)
    finally:
        dd.setWorkspace(None)
    assert float(((total - want).norm() / want.norm()).item()) <= 1e-5
