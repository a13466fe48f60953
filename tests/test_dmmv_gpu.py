"""GPU parity of the decode dequant-matvec family, through the C ABI, against the CPU oracle.

Bars: dequantised weights bit-exact; f32 outputs relative L2 <= 1e-4 against the
f64-accumulated oracle; the reference's own kernel-test fixtures within the absolute
tolerances those tests use (src/compute/forward_metal.zig:11331, 11407, 11496, 11578).
"""
import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import synth
from helpers import canary_intact, dev, dev_padded, out_with_canary, rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-4  # relative L2 bar for f32 outputs
ALL_TYPES = [zb.Q4_K, zb.Q5_K, zb.Q6_K, zb.Q8_0, zb.MXFP4, zb.Q5_0, zb.Q5_1, zb.F16, zb.F32]
IDS = [zb.TYPE_NAMES[t] for t in ALL_TYPES]


def k_for(t, blocks):
    return max(zb.block_size(t), 32) * blocks if zb.block_size(t) > 1 else 32 * blocks


@pytest.mark.parametrize("t", ALL_TYPES, ids=IDS)
def test_dequant_rows_bit_exact(gpu, oracle, t):
    torch, ctx, dd = gpu
    g = synth.rng(100, t)
    M, K = 37, k_for(t, 3)
    w = synth.quant_matrix(g, t, M, K)
    wd = dev(torch, w)
    out = torch.empty(M * K, dtype=torch.float32, device="cuda")
    dd.dequantRows(t, wd, out, 0, M, K)
    ctx.submit_and_wait()
    want = oracle.dequant_rows(w, M, K, t)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.reshape(-1).view(np.uint32))
    # a row range with a byte offset
    out2 = torch.empty(5 * K, dtype=torch.float32, device="cuda")
    rb = zb.row_bytes(t, K)
    dd.dequantRows(t, wd, out2, 3, 5, K, a_offset=2 * rb)
    ctx.submit_and_wait()
    assert np.array_equal(out2.cpu().numpy().view(np.uint32), want[5:10].reshape(-1).view(np.uint32))


def test_dequant_edge_bytes_bit_exact(gpu, oracle):
    """All-ones / all-zero quant bytes, extreme scales, MXFP4 e=0 and e=254."""
    torch, ctx, dd = gpu
    for t in (zb.Q4_K, zb.Q5_K, zb.Q6_K, zb.Q8_0, zb.MXFP4, zb.Q5_0, zb.Q5_1):
        bs, bpb = synth.BLOCK[t]
        blocks = np.zeros((4, bpb), np.uint8)
        blocks[1] = 0xFF
        blocks[2] = np.arange(bpb) * 37 & 0xFF
        blocks[3] = 0x80
        # keep f16 fields finite
        h = np.array([6.1e-5], np.float16).view(np.uint8)
        for b in (1, 2, 3):
            if t in (zb.Q4_K, zb.Q5_K):
                blocks[b, 0:2] = h
                blocks[b, 2:4] = np.array([65504.0], np.float16).view(np.uint8)
            elif t == zb.Q6_K:
                blocks[b, 208:210] = np.array([-0.5], np.float16).view(np.uint8)
            elif t in (zb.Q8_0, zb.Q5_0, zb.Q5_1):
                blocks[b, 0:2] = h
                if t == zb.Q5_1:
                    blocks[b, 2:4] = np.array([-3.0], np.float16).view(np.uint8)
        if t == zb.MXFP4:
            blocks[0, 0], blocks[1, 0], blocks[3, 0] = 0, 254, 1
        K = bs * 4
        w = blocks.reshape(-1)
        out = torch.empty(K, dtype=torch.float32, device="cuda")
        dd.dequantRows(t, dev(torch, w), out, 0, 1, K)
        ctx.submit_and_wait()
        want = oracle.dequant_rows(w, 1, K, t)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.reshape(-1).view(np.uint32)), zb.TYPE_NAMES[t]


@pytest.mark.parametrize("t", ALL_TYPES, ids=IDS)
@pytest.mark.parametrize("M,blocks", [(1, 1), (2, 1), (67, 5), (513, 16)])
def test_dmmv_matches_oracle(gpu, oracle, t, M, blocks):
    torch, ctx, dd = gpu
    K = k_for(t, blocks)
    g = synth.rng(101, t * 1000 + M)
    w = synth.quant_matrix(g, t, M, K)
    x = synth.activations(g, K)
    y = out_with_canary(torch, M)
    dd.recordDispatch(t, dev(torch, w), dev(torch, x), y, M, K)
    ctx.submit_and_wait()
    want = oracle.dmmv_f64(w, t, M, K, x)
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy(), want) <= TOL


@pytest.mark.parametrize("t", ALL_TYPES, ids=IDS)
def test_dmmv_offsets_acc_mode_and_poison(gpu, oracle, t):
    """Non-zero a/x/y offsets, acc_mode 1, 0xA5-poisoned padding either side, canaries after y."""
    torch, ctx, dd = gpu
    M, K = 131, k_for(t, 4)
    g = synth.rng(102, t)
    w = synth.quant_matrix(g, t, M, K)
    x = synth.activations(g, K)
    y0 = synth.activations(g, M)
    rb = zb.row_bytes(t, K)
    # weight offset: one whole matrix of poison in front (as forward_metal.zig:11424-11433 does)
    a_off = M * rb
    a_off += (-a_off) % 16 if t in (zb.Q4_K, zb.Q5_K) else 0
    wd, _ = dev_padded(torch, w, front=a_off, back=64)
    xd = torch.full((K + 8 + 4,), float("nan"), dtype=torch.float32, device="cuda")
    xd[8:8 + K] = dev(torch, x)
    y = out_with_canary(torch, 3 + M)
    y[3:3 + M] = dev(torch, y0)
    dd.recordDispatch(t, wd, xd, y, M, K, a_offset=a_off, x_offset=32, y_offset=12, acc_mode=1)
    ctx.submit_and_wait()
    want = oracle.dmmv_f64(w, t, M, K, x) + y0.astype(np.float64)
    got = y.cpu().numpy()
    assert np.all(got[:3] == 0.0) and canary_intact(y, 3 + M)
    assert rel_l2(got[3:3 + M], want) <= TOL
    # acc_mode 0 overwrites
    dd.recordDispatch(t, wd, xd, y, M, K, a_offset=a_off, x_offset=32, y_offset=12, acc_mode=0)
    ctx.submit_and_wait()
    assert rel_l2(y[3:3 + M].cpu().numpy(), oracle.dmmv_f64(w, t, M, K, x)) <= TOL


def test_dmmv_unaligned_kquant_base(gpu, oracle):
    """Q4_K / Q5_K weights at a 4-byte (not 16-byte) aligned offset take the word-load path."""
    torch, ctx, dd = gpu
    for t in (zb.Q4_K, zb.Q5_K):
        M, K = 19, 768
        g = synth.rng(103, t)
        w = synth.quant_matrix(g, t, M, K)
        x = synth.activations(g, K)
        wd, off = dev_padded(torch, w, front=4, back=64)
        y = out_with_canary(torch, M)
        dd.recordDispatch(t, wd, dev(torch, x), y, M, K, a_offset=off)
        ctx.submit_and_wait()
        assert rel_l2(y[:M].cpu().numpy(), oracle.dmmv_f64(w, t, M, K, x)) <= TOL


def test_reference_fixture_q5k_many_rows(gpu, oracle):
    # src/compute/forward_metal.zig:11411-11498: M=257, K=512, a_offset = one matrix, 0xCD poison, abs tol 0.05
    torch, ctx, dd = gpu
    w, x = synth.pattern_q5k()
    M, K = 257, 512
    wd, off = dev_padded(torch, w, front=w.size, back=0, fill=0xCD)
    y = out_with_canary(torch, M)
    dd.recordDispatch(zb.Q5_K, wd, dev(torch, x), y, M, K, a_offset=off)
    ctx.submit_and_wait()
    want = oracle.dmmv_f32seq(w, zb.Q5_K, M, K, x)
    assert np.max(np.abs(y[:M].cpu().numpy() - want)) <= 0.05


def test_reference_fixture_q6k_many_rows(gpu, oracle):
    # src/compute/forward_metal.zig:11500-11580
    torch, ctx, dd = gpu
    w, x = synth.pattern_q6k()
    M, K = 257, 512
    wd, off = dev_padded(torch, w, front=w.size, back=2, fill=0xCD)
    y = out_with_canary(torch, M)
    dd.recordDispatch(zb.Q6_K, wd, dev(torch, x), y, M, K, a_offset=off)
    ctx.submit_and_wait()
    want = oracle.dmmv_f32seq(w, zb.Q6_K, M, K, x)
    assert np.max(np.abs(y[:M].cpu().numpy() - want)) <= 0.05


def test_reference_fixture_q5k_3010_and_mxfp4_48(gpu):
    # src/compute/forward_metal.zig:11293-11331 and 14238-14303
    torch, ctx, dd = gpu
    b = np.zeros(176, np.uint8)
    b[0:2] = np.array([1.0], np.float16).view(np.uint8)
    b[4], b[5], b[48] = 1, 1, 0x3A
    x = np.zeros(256, np.float32)
    x[0], x[1], x[32] = 1.0, 100.0, 1000.0
    y = out_with_canary(torch, 1)
    dd.recordDispatch(zb.Q5_K, dev(torch, b), dev(torch, x), y, 1, 256)
    ctx.submit_and_wait()
    assert abs(float(y[0]) - 3010.0) <= 0.001
    rows = np.tile(np.concatenate([[127], np.full(16, 0x42)]).astype(np.uint8), 4)
    y = out_with_canary(torch, 4)
    dd.recordDispatch(zb.MXFP4, dev(torch, rows), dev(torch, np.ones(32, np.float32)), y, 4, 32)
    ctx.submit_and_wait()
    assert np.allclose(y[:4].cpu().numpy(), 48.0, atol=0.01)


@pytest.mark.parametrize("t", [zb.Q4_K, zb.Q8_0, zb.Q6_K, zb.MXFP4], ids=["q4_k", "q8_0", "q6_k", "mxfp4"])
def test_fused_gate_up_swiglu(gpu, oracle, t):
    # out[r] = silu(Wg[r].x) * (Wu[r].x)  (src/shaders/dmmv_q4k_fused_gate_up_swiglu.comp:195-218)
    torch, ctx, dd = gpu
    M, K = 301, k_for(t, 6)
    g = synth.rng(104, t)
    wg, wu = synth.quant_matrix(g, t, M, K), synth.quant_matrix(g, t, M, K)
    x = synth.activations(g, K) * 0.05  # keep silu away from saturation
    out = out_with_canary(torch, M)
    dd.dispatchDmmvFusedGateUpSwiglu(t, dev(torch, wg), dev(torch, wu), dev(torch, x), out, M, K)
    ctx.submit_and_wait()
    gate = oracle.dmmv_f64(wg, t, M, K, x)
    up = oracle.dmmv_f64(wu, t, M, K, x)
    want = gate / (1.0 + np.exp(-gate)) * up
    assert canary_intact(out, M)
    assert rel_l2(out[:M].cpu().numpy(), want) <= TOL


@pytest.mark.parametrize("t", [zb.Q8_0, zb.Q4_K], ids=["q8_0", "q4_k"])
def test_sigmoid_acc(gpu, oracle, t):
    # y[r] += sigmoid(g[idx]) * (W[r].x)  (src/shaders/dmmv_q8_0_sigmoid_acc.comp:95-132)
    torch, ctx, dd = gpu
    M, K = 77, k_for(t, 8)
    g = synth.rng(105, t)
    w = synth.quant_matrix(g, t, M, K)
    x = synth.activations(g, K)
    y0 = synth.activations(g, M)
    gate = np.array([9.0, -0.7, 3.0], np.float32)
    y = out_with_canary(torch, M)
    y[:M] = dev(torch, y0)
    dd.dispatchDmmvSigmoidAcc(t, dev(torch, w), dev(torch, x), y, dev(torch, gate), M, K, gate_index=1)
    ctx.submit_and_wait()
    want = y0 + oracle.dmmv_f64(w, t, M, K, x) / (1.0 + np.exp(0.7))
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy(), want) <= TOL


def test_linearity_at_full_size(gpu):
    """Config-1 size (4096 x 4096 Q4_K) and the LM-head shape: W(a x1 + b x2) = a W x1 + b W x2."""
    torch, ctx, dd = gpu
    for t, M, K in ((zb.Q4_K, 4096, 4096), (zb.Q6_K, 151936, 4096)):
        w = synth.torch_quant_matrix(t, M, K, "cuda", seed=5)
        gen = torch.Generator(device="cuda").manual_seed(6)
        x1 = torch.randn(K, device="cuda", generator=gen)
        x2 = torch.randn(K, device="cuda", generator=gen)
        ys = [torch.empty(M, device="cuda") for _ in range(3)]
        for xv, yv in zip((x1, x2, (0.5 * x1 - 2.0 * x2).contiguous()), ys):
            dd.recordDispatch(t, w, xv, yv, M, K)
        ctx.submit_and_wait()
        want = 0.5 * ys[0].double() - 2.0 * ys[1].double()
        for i, yv in enumerate(ys):
            assert bool(torch.isfinite(yv).all()), f"{zb.TYPE_NAMES[t]}: dispatch {i} left non-finite rows"
        err = (ys[2].double() - want).norm() / want.norm()
        assert float(err) <= TOL, zb.TYPE_NAMES[t]


def test_full_size_rows_match_oracle_sample(gpu, oracle):
    """Config-1 shape: a sample of rows of the 4096 x 4096 Q4_K product against the oracle."""
    torch, ctx, dd = gpu
    M = K = 4096
    g = synth.rng(1, 0)
    w = synth.quant_matrix(g, zb.Q4_K, M, K)
    x = synth.activations(g, K)
    y = out_with_canary(torch, M)
    dd.recordDispatch(zb.Q4_K, dev(torch, w), dev(torch, x), y, M, K)
    ctx.submit_and_wait()
    want = oracle.dmmv_f64(w, zb.Q4_K, M, K, x)
    assert rel_l2(y[:M].cpu().numpy(), want) <= TOL


def test_error_codes(gpu):
    """UnsupportedQuantType / InvalidArgument as the reference raises them (src/compute/dmmv.zig:822, 767)."""
    torch, ctx, dd = gpu
    w = torch.zeros(144 * 4, dtype=torch.uint8, device="cuda")
    x = torch.zeros(256, device="cuda")
    y = torch.zeros(4, device="cuda")
    with pytest.raises(zb.UnsupportedQuantType):
        dd.recordDispatch(10, w, x, y, 4, 256)  # q2_k has no kernel
    with pytest.raises(zb.InvalidArgument):
        dd.recordDispatch(zb.Q4_K, w, x, y, 4, 200)  # K not a multiple of 256
    with pytest.raises(zb.InvalidArgument):
        dd.recordDispatch(zb.Q4_K, w, x, y, 5, 256)  # weights out of range
    with pytest.raises(zb.InvalidArgument):
        dd.recordDispatch(zb.Q4_K, w, x, y, 4, 256, x_offset=4)  # x not 16-byte aligned / out of range
    with pytest.raises(zb.InvalidArgument):
        dd.recordDispatch(zb.Q4_K, w, x, y, 4, 256, y_offset=8)  # y out of range
    with pytest.raises(zb.InvalidArgument):
        dd.recordDispatch(zb.Q4_K, w, x, y, 0, 256)
    # the context stays usable after errors
    dd.recordDispatch(zb.Q4_K, w, x, y, 4, 256)
    ctx.submit_and_wait()
    assert float(y.abs().sum()) == 0.0


@pytest.mark.parametrize("t", [zb.Q4_K, zb.Q6_K], ids=["q4_k", "q6_k"])
@pytest.mark.parametrize("M,K", [(16, 2048), (67, 2048), (300, 6144), (1000, 12288), (4099, 4096), (33, 14336),
                                 (2048, 512), (4096, 3072), (300, 1536), (4100, 768)])
def test_streaming_shapes(gpu, oracle, t, M, K):
    """Shapes that take the split-K streaming kernels (rows not a multiple of 16, tiles split across
    workers inside a CTA and across CTAs, K up to the shared-memory limit, Q6_K rows that are not
    16-byte aligned because K is not a multiple of 2048) and one beyond the limit."""
    torch, ctx, dd = gpu
    g = synth.rng(106, t * 100000 + M * 31 + K)
    w = synth.quant_matrix(g, t, M, K)
    x = synth.activations(g, K) * np.float32(3.0 if M % 2 else 1e-3)  # also exercise the per-block scaling
    y0 = synth.activations(g, M)
    y = out_with_canary(torch, M)
    y[:M] = dev(torch, y0)
    wd, xd = dev(torch, w), dev(torch, x)
    dd.recordDispatch(t, wd, xd, y, M, K, acc_mode=1)
    ctx.submit_and_wait()
    want = oracle.dmmv_f64(w, t, M, K, x)
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy() - y0, want) <= TOL
    # twice in a row: the split-K hand-off state must be clean after a launch
    for _ in range(2):
        dd.recordDispatch(t, wd, xd, y, M, K, acc_mode=0)
    ctx.submit_and_wait()
    assert rel_l2(y[:M].cpu().numpy(), want) <= TOL


def test_streaming_extreme_activations(gpu, oracle):
    """Activation blocks that are all zero, tiny, huge, or mixed by 2^40 within a block."""
    torch, ctx, dd = gpu
    M, K = 48, 4096
    g = synth.rng(107, 0)
    x = synth.activations(g, K)
    x[0:256] = 0.0
    x[256:512] *= np.float32(1e-30)
    x[512:768] *= np.float32(1e30)
    x[768:1024:2] *= np.float32(2.0 ** -40)
    for t in (zb.Q4_K, zb.Q6_K):
        w = synth.quant_matrix(g, t, M, K)
        y = out_with_canary(torch, M)
        dd.recordDispatch(t, dev(torch, w), dev(torch, x), y, M, K)
        ctx.submit_and_wait()
        assert rel_l2(y[:M].cpu().numpy(), oracle.dmmv_f64(w, t, M, K, x)) <= TOL


@pytest.mark.parametrize("t,Ms,K", [(zb.Q4_K, (4096, 1024, 1024), 4096), (zb.Q4_K, (1000, 37), 2048),
                                   (zb.Q4_K, (16, 16, 48), 512), (zb.Q6_K, (64, 32, 32), 2048),
                                   (zb.Q8_0, (40, 24), 256)],
                         ids=["q4k_qkv", "q4k_ragged_pair", "q4k_tiny", "q6k_fallback", "q8_0_fallback"])
def test_dispatch_multi(gpu, oracle, t, Ms, K):
    """Grouped matvec (the Q, K, V dispatches of one token as one call) against the oracle, twice in
    a row, with accumulate mode on the second call."""
    torch, ctx, dd = gpu
    g = synth.rng(108, t * 1000 + sum(Ms))
    ws = [synth.quant_matrix(g, t, M, K) for M in Ms]
    x = synth.activations(g, K)
    xd = dev(torch, x)
    wds = [dev(torch, w) for w in ws]
    ys = [out_with_canary(torch, M) for M in Ms]
    dd.recordDispatchMulti(t, wds, xd, ys, list(Ms), K)
    dd.recordDispatchMulti(t, wds, xd, ys, list(Ms), K, acc_mode=1)
    ctx.submit_and_wait()
    for w, M, y in zip(ws, Ms, ys):
        assert canary_intact(y, M)
        assert rel_l2(y[:M].cpu().numpy(), 2.0 * oracle.dmmv_f64(w, t, M, K, x)) <= TOL


@pytest.mark.parametrize("M,K", [(64, 2880), (300, 2880), (2880, 2880), (100, 512), (48, 1056), (1000, 8192)])
def test_streaming_mxfp4(gpu, oracle, M, K):
    """MXFP4 shapes that take the streaming kernel: 17-byte blocks, rows that are only 2-byte aligned,
    K not a multiple of 256, ragged row tiles, the last piece at the very end of the buffer, scale
    byte 0, overwrite and accumulate, twice in a row."""
    torch, ctx, dd = gpu
    g = synth.rng(109, M * 7 + K)
    w = synth.quant_matrix(g, zb.MXFP4, M, K).copy()
    wb = w.reshape(M, K // 32, 17)
    wb[::3, ::5, 0] = 0          # E8M0 byte 0 (2^-127)
    wb[1::4, 1::7, 0] = 127 + 3  # larger scales
    x = synth.activations(g, K) * np.float32(2.0 if M % 2 else 1e-2)
    y0 = synth.activations(g, M)
    y = out_with_canary(torch, M)
    y[:M] = dev(torch, y0)
    wd, xd = dev(torch, w), dev(torch, x)
    dd.recordDispatch(zb.MXFP4, wd, xd, y, M, K, acc_mode=1)
    ctx.submit_and_wait()
    want = oracle.dmmv_f64(w, zb.MXFP4, M, K, x)
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy() - y0, want) <= TOL
    for _ in range(2):
        dd.recordDispatch(zb.MXFP4, wd, xd, y, M, K, acc_mode=0)
    ctx.submit_and_wait()
    assert rel_l2(y[:M].cpu().numpy(), want) <= TOL
    # weights at a 16-byte offset inside a poisoned buffer
    wpad, off = dev_padded(torch, w, front=48, back=16)
    y2 = out_with_canary(torch, M)
    dd.recordDispatch(zb.MXFP4, wpad, xd, y2, M, K, a_offset=off)
    ctx.submit_and_wait()
    assert rel_l2(y2[:M].cpu().numpy(), want) <= TOL


@pytest.mark.parametrize("t,M,K,n_heads,nc,sink", [
    (zb.Q4_K, 4096, 4096, 32, 4, "some"),    # streaming kernel: merged while the activation is loaded
    (zb.Q4_K, 4096, 4096, 32, 1, None),
    (zb.Q4_K, 2048, 2048, 16, 3, "all"),
    (zb.Q4_K, 200, 1024, 8, 4, "some"),      # small matrix: merge kernel, then one warp per row
    (zb.Q6_K, 512, 1024, 4, 6, "none"),      # another type, more chunks than the fused path takes
])
def test_o_proj_merge(gpu, oracle, t, M, K, n_heads, nc, sink):
    """Split-K flash-attention merge fused with the O projection (src/shaders/dmmv_q4k_o_proj_merge.comp): chunks
    with zero weight, heads with and without a sink (NaN = none), accumulate into the hidden vector."""
    torch, ctx, dd = gpu
    hd = K // n_heads
    g = synth.rng(330, M + nc)
    w = synth.quant_matrix(g, t, M, K)
    part = synth.activations(g, n_heads * nc * hd)
    mx = (synth.activations(g, n_heads, nc) * np.float32(3.0)).astype(np.float32)
    ls = (g.random((n_heads, nc)).astype(np.float32) * np.float32(50.0) + np.float32(0.5))
    if nc > 1:
        ls[1, nc - 1] = 0.0   # a chunk that saw no keys
    lse = np.stack([mx, ls], axis=-1).reshape(-1)
    buf = np.concatenate([part, lse]).astype(np.float32)
    sinks = None
    if sink is not None:
        sinks = np.full(n_heads + 5, np.nan, np.float32)
        if sink in ("some", "all"):
            sinks[5:] = synth.activations(g, n_heads) * np.float32(2.0)
        if sink == "some":
            sinks[5 + 1::2] = np.nan
    x = oracle.attn_merge(buf, sinks, n_heads, nc, hd, 5 if sinks is not None else 0)
    h0 = synth.activations(g, M)
    y = out_with_canary(torch, M)
    y[:M] = dev(torch, h0)
    dd.dispatchDmmvOprojMerge(t, dev(torch, w), dev(torch, buf), None if sinks is None else dev(torch, sinks), y, M, K,
                              n_heads, nc, 5 if sinks is not None else 0, hd)
    ctx.submit_and_wait()
    want = oracle.dmmv_f64(w, t, M, K, x)
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy() - h0, want) <= 1e-4
    with pytest.raises(zb.InvalidArgument):
        dd.dispatchDmmvOprojMerge(t, dev(torch, w), dev(torch, buf), None, y, M, K, n_heads + 1, nc, 0, hd)
