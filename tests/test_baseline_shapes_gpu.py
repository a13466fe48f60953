"""GPU parity at the benchmark configurations' own shapes.

The small-shape tests pin every kernel against the full oracle product; these run the kernels the
benchmark runs, at the sizes it runs them (longest K loops, most tiles, split-K and variant choices the
real shapes trigger), and compare with the oracle on a sample the CPU finishes in seconds:
  prefill dequant-GEMM: Q4_K 12288 x 4096, Q6_K 4096 x 12288 at T = 128 / 512 / 2048 and MXFP4 5760 x 2880:
    >= 64 sampled weight rows x every token (bar 5e-3, bf16 tensor cores);
  grouped MoE prefill: 256 experts top-8 (gate / up 512 x 2048 Q4_K, down 2048 x 512 Q6_K) at T = 512 and 32
    experts top-4 (2880 x 2880 MXFP4) at T = 1024: sampled (token, slot) pairs against the oracle, and every
    pair against the library's own per-pair f32 kernel;
  one MoE decode layer pair of each configuration against the oracle-composed sequence, biases included.
Weights are generated on the device (as the benchmark does) and copied back for the oracle.
"""
import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import synth
from zinc_b200.moe_step import GPT_OSS_MOE, QWEN35_MOE, MoeDecode
from helpers import canary_intact, dev, oracle_moe_decode_layer, out_with_canary, rel_l2

pytestmark = pytest.mark.gpu
TOL_TC = 5e-3   # bf16 operands on the tensor cores
TOL = 1e-4      # f32 paths


def _rows_sample(g, M, n):
    rows = np.unique(np.concatenate([[0, 1, 127, 128, M - 129, M - 128, M - 1], g.integers(0, M, size=n)]))
    return rows.astype(np.int64)


@pytest.mark.parametrize("T", [128, 512, 2048])
@pytest.mark.parametrize("t,M,K", [(zb.Q4_K, 12288, 4096), (zb.Q6_K, 4096, 12288), (zb.MXFP4, 5760, 2880)],
                         ids=["q4_k_12288x4096", "q6_k_4096x12288", "mxfp4_5760x2880"])
def test_prefill_gemm_config_shapes(gpu, oracle, t, M, K, T):
    torch, ctx, dd = gpu
    g = synth.rng(3, t * 10000 + T)
    W = synth.torch_quant_matrix(t, M, K, "cuda:0", 900 + t)
    Xf = synth.activations(g, T, K)
    bits = synth.to_bf16_bits(Xf.reshape(-1))
    Xb = synth.bf16_bits_to_f32(bits).reshape(T, K)
    D = out_with_canary(torch, T * M)
    dd.recordMulMm(t, W, dev(torch, bits.view(np.int16)), D, M, T, K, K, M, 0, 0, 0, zb.BF16)
    ctx.submit_and_wait()
    assert canary_intact(D, T * M)
    got = D[:T * M].view(T, M)
    assert bool(torch.isfinite(got).all().item())
    rows = _rows_sample(g, M, 64)
    rb = zb.row_bytes(t, K)
    wsub = W.view(M, rb)[torch.from_numpy(rows).cuda()].contiguous().cpu().numpy().reshape(-1)
    want = oracle.gemm_f64(wsub, t, len(rows), K, Xb)                   # [T][rows]
    have = got[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    assert rel_l2(have, want) <= (1e-5 if t == zb.MXFP4 else TOL_TC)
    assert max(rel_l2(have[i], want[i]) for i in range(0, T, max(1, T // 64))) <= 2e-2
    # every row of the output took part: column norms of the whole product are in a sane band
    norms = got.float().norm(dim=0)
    assert float(norms.min().item()) > 0.0


def _moe_prefill_case(gpu, oracle, S, T, n_sample):
    torch, ctx, dd = gpu
    E, k, H, F = S.n_experts, S.top_k, S.hidden, S.ffn
    g = synth.rng(4 if S is QWEN35_MOE else 5, T)
    Wg = synth.torch_quant_matrix(S.t_gate_up, E * F, H, "cuda:0", 811)
    Wd = synth.torch_quant_matrix(S.t_down, E * H, F, "cuda:0", 813)
    sg, sd = zb.expert_slice_bytes(S.t_gate_up, F, H), zb.expert_slice_bytes(S.t_down, H, F)
    X = synth.activations(g, T, H)
    logits = synth.activations(g, T, E)
    routing = torch.zeros(T * 2 * k, dtype=torch.int32, device="cuda")
    dd.dispatchSoftmaxTopk(dev(torch, logits), routing, E, k, S.rule, T)
    ctx.submit_and_wait()
    ids_d = routing.view(T, 2 * k)[:, :k].contiguous()
    ids = ids_d.cpu().numpy().astype(np.uint32)
    A = synth.activations(g, T * k, F)        # stands in for the activation rows the down projection reads
    Xd, Ad = dev(torch, X), dev(torch, A)
    ws = torch.empty(max(dd.moeGroupedWorkspaceBytes(T, k, H, E), dd.moeGroupedWorkspaceBytes(T * k, 1, F, E)),
                     dtype=torch.uint8, device="cuda")
    out = {}
    for path in ("grouped", "per_pair"):
        dd.setWorkspace(ws if path == "grouped" else None)
        try:
            Yg = out_with_canary(torch, T * k * F)
            Yd = out_with_canary(torch, T * k * H)
            n0 = ctx.launch_count
            dd.recordMoeBatchedDispatch(S.t_gate_up, Wg, Xd, Yg, ids_d, F, H, sg, E, k, T, H, k * F)
            dd.recordMoeBatchedDispatch(S.t_down, Wd, Ad, Yd, ids_d, H, F, sd, E, 1, T * k, F, H)
            ctx.submit_and_wait()
            launches = ctx.launch_count - n0
        finally:
            dd.setWorkspace(None)
        assert canary_intact(Yg, T * k * F) and canary_intact(Yd, T * k * H)
        assert launches == (6 if path == "grouped" else 2), "the grouped path must be the one that ran"
        out[path] = (Yg[:T * k * F].view(T, k, F), Yd[:T * k * H].view(T * k, H))
    # every pair: tensor-core path against the library's f32 per-pair kernel
    for a, b in zip(out["grouped"], out["per_pair"]):
        num = float((a.double() - b.double()).norm().item())
        assert num / float(b.double().norm().item()) <= TOL_TC
    # sampled pairs against the oracle (both paths)
    wg_h, wd_h = Wg.cpu().numpy(), Wd.cpu().numpy()
    toks = g.integers(0, T, size=n_sample)
    slots = g.integers(0, k, size=n_sample)
    for path, tol in (("grouped", TOL_TC), ("per_pair", TOL)):
        Yg, Yd = out[path]
        hg, wgt, hd, wdn = [], [], [], []
        for tok, sl in zip(toks, slots):
            e = np.array([ids[tok, sl]], np.uint32)
            wgt.append(oracle.moe_dmmv_f64(wg_h, S.t_gate_up, F, H, sg, e, H, X[tok:tok + 1])[0])
            hg.append(Yg[tok, sl].cpu().numpy())
            p = tok * k + sl
            wdn.append(oracle.moe_dmmv_f64(wd_h, S.t_down, H, F, sd, e, F, A[p:p + 1])[0])
            hd.append(Yd[p].cpu().numpy())
        assert rel_l2(np.stack(hg), np.stack(wgt)) <= tol
        assert rel_l2(np.stack(hd), np.stack(wdn)) <= tol


def test_moe_prefill_qwen35_shape(gpu, oracle):
    # 256 experts, top-8, T = 512: 4096 pairs, 32-pair tiles, gate / up 512 x 2048 Q4_K, down 2048 x 512 Q6_K
    _moe_prefill_case(gpu, oracle, QWEN35_MOE, 512, 96)


def test_moe_prefill_gpt_oss_shape(gpu, oracle):
    # 32 experts, top-4, T = 1024: 4096 pairs, 128-pair tiles, 2880 x 2880 MXFP4 (1530-byte rows)
    _moe_prefill_case(gpu, oracle, GPT_OSS_MOE, 1024, 48)


@pytest.mark.parametrize("name", ["qwen35", "gpt_oss"])
def test_moe_decode_layers_against_oracle(gpu, oracle, name):
    """Two full-size MoE decode layers through the op sequence the benchmark records, against the
    oracle-composed sequence (router -> top-k -> gate / up (+ biases) -> activation -> down (+ bias) ->
    weighted sum -> shared expert)."""
    import dataclasses

    torch, ctx, dd = gpu
    shape = dataclasses.replace(QWEN35_MOE if name == "qwen35" else GPT_OSS_MOE, n_layers=2)
    step = MoeDecode.build(torch, dd, shape, seed=11)
    step.record()
    ctx.submit_and_wait()
    got = step.hidden.cpu().numpy().astype(np.float64)
    x = step.x.cpu().numpy()
    want = np.zeros(shape.hidden, np.float64)
    cpu = lambda t: None if t is None else t.cpu().numpy()
    for w in step.layers:
        contrib, _ = oracle_moe_decode_layer(oracle, x, cpu(w.router), cpu(w.wg), cpu(w.wu), cpu(w.wd), shape, shape.ffn,
                                             router_bias=cpu(w.router_bias), bg=cpu(w.bg), bu=cpu(w.bu), bd=cpu(w.bd),
                                             sg=cpu(w.sg), su=cpu(w.su), sd=cpu(w.sd))
        want += contrib
    assert rel_l2(got, want) <= TOL


def test_bias_entry_points(gpu, oracle):
    # zc_bias_add (src/shaders/bias_add.comp) and the per-slot fused forms against plain numpy
    torch, ctx, dd = gpu
    g = synth.rng(6, 0)
    E, M, k, H = 7, 301, 3, 129
    gate, up = synth.activations(g, k, M) * 3, synth.activations(g, k, M) * 3
    bg, bu, bd = synth.activations(g, E, M), synth.activations(g, E, M), synth.activations(g, E, H)
    ids = np.array([6, 0, 3], np.uint32)
    wts = np.array([0.5, 0.3, 0.2], np.float32)
    routing = dev(torch, np.concatenate([ids, wts.view(np.uint32)]))
    for oai in (False, True):
        y = out_with_canary(torch, k * M)
        dd.dispatchMoeBiasAct(dev(torch, gate), dev(torch, up), dev(torch, bg), dev(torch, bu), routing, y, M, k, E, oai=oai)
        ctx.submit_and_wait()
        want = oracle.swiglu((gate + bg[ids]).reshape(-1), (up + bu[ids]).reshape(-1), oai=oai)
        assert canary_intact(y, k * M) and rel_l2(y[:k * M].cpu().numpy(), want) <= 1e-6
    h0 = synth.activations(g, H)
    a = out_with_canary(torch, H)
    a[:H] = dev(torch, h0)
    dd.dispatchMoeWeightedBiasAcc(a, dev(torch, bd), routing, H, k, E)
    ctx.submit_and_wait()
    assert canary_intact(a, H)
    assert rel_l2(a[:H].cpu().numpy(), h0 + (wts[:, None] * bd[ids]).sum(0)) <= 1e-6
    # the reference's own form: one slice of a bias tensor onto one expert's vector
    v = out_with_canary(torch, M)
    v[:M] = dev(torch, gate[1])
    dd.dispatchBiasAddSlice(v, dev(torch, bg.reshape(-1)), 3 * M, M)
    ctx.submit_and_wait()
    assert canary_intact(v, M) and np.array_equal(v[:M].cpu().numpy(), gate[1] + bg[3])
    with pytest.raises(zb.InvalidArgument):
        dd.dispatchBiasAddSlice(v, dev(torch, bg.reshape(-1)), E * M - 5, M)   # slice runs past the bias tensor


def test_bad_expert_id_is_reported_not_followed(gpu, oracle):
    """An id beyond the experts the buffer holds never becomes an address: the call completes, and
    zc_submit_and_wait reports it; the context keeps working afterwards."""
    torch, ctx, dd = gpu
    t, E, M, K, n_used = zb.Q4_K, 3, 64, 512, 2
    g = synth.rng(7, 0)
    w = synth.quant_matrix(g, t, E * M, K)
    stride = zb.expert_slice_bytes(t, M, K)
    x = synth.activations(g, 1, K)
    wd, xd = dev(torch, w), dev(torch, x)
    for ids in ([1, 3], [0xFFFFFFF0, 2]):
        r = dev(torch, np.concatenate([np.array(ids, np.uint32), np.ones(n_used, np.float32).view(np.uint32)]))
        y = out_with_canary(torch, n_used * M)
        dd.recordMoeDispatch(t, wd, xd, y, r, M, K, stride, n_used, 0)
        with pytest.raises(zb.InvalidArgument):
            ctx.submit_and_wait()
        assert canary_intact(y, n_used * M)
        h = out_with_canary(torch, M)
        dd.dispatchMoeFusedDownAcc(t, wd, dev(torch, np.repeat(x, n_used, axis=0)), h, r, M, K, stride, n_used, K)
        with pytest.raises(zb.InvalidArgument):
            ctx.submit_and_wait()
    good = dev(torch, np.concatenate([np.array([2, 0], np.uint32), np.ones(n_used, np.float32).view(np.uint32)]))
    y = out_with_canary(torch, n_used * M)
    dd.recordMoeDispatch(t, wd, xd, y, good, M, K, stride, n_used, 0)
    ctx.submit_and_wait()
    want = oracle.moe_dmmv_f64(w, t, M, K, stride, np.array([2, 0], np.uint32), K, np.repeat(x, n_used, axis=0))
    assert rel_l2(y[:n_used * M].cpu().numpy(), want) <= TOL
