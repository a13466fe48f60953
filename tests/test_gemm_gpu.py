"""GPU parity of the batched-prefill paths (zc_dmmv_batch, zc_mul_mm) against the f64 oracle.

Bars: f32-activation paths relative L2 <= 1e-4 when they keep f32 precision; the bf16
tensor-core path <= 5e-3 against the exact product and <= 4e-3 against the oracle evaluated
on bf16-rounded operands (the tensor-core kernel also rounds d*sc and dmin*m to bf16 before it
forms a weight, which the rounded-operand oracle does not).
"""
import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import synth
from helpers import canary_intact, dev, out_with_canary, rel_l2

pytestmark = pytest.mark.gpu
TOL_F32, TOL_BF16, TOL_BF16_OPERANDS = 1e-4, 5e-3, 4e-3


@pytest.mark.parametrize("t", [zb.Q4_K, zb.Q6_K, zb.Q5_K, zb.Q8_0, zb.MXFP4],
                         ids=["q4_k", "q6_k", "q5_k", "q8_0", "mxfp4"])
@pytest.mark.parametrize("cols", [1, 5, 40, 129])
def test_dmmv_batch(gpu, oracle, t, cols):
    # Y[c][M] = W X[c][K]  (src/compute/dmmv.zig:880-926; layouts src/compute/forward.zig:8141-8146)
    torch, ctx, dd = gpu
    M = 96 + 7
    K = 512 if zb.block_size(t) == 256 else 160
    g = synth.rng(300, t * 1000 + cols)
    w = synth.quant_matrix(g, t, M, K)
    X = synth.activations(g, cols, K)
    Y = out_with_canary(torch, cols * M)
    dd.recordBatchDispatchPush(t, dev(torch, w), dev(torch, X), Y, M, K, 0, 0, 0, cols)
    ctx.submit_and_wait()
    got = Y[:cols * M].cpu().numpy().reshape(cols, M)
    exact = oracle.gemm_f64(w, t, M, K, X)
    assert canary_intact(Y, cols * M)
    e = rel_l2(got, exact)
    if e > TOL_F32:  # tensor-core path: compare with the bf16-operand product
        assert e <= TOL_BF16
        assert rel_l2(got, oracle.gemm_f64(w, t, M, K, X, round_bf16=True)) <= TOL_BF16_OPERANDS


@pytest.mark.parametrize("t", [zb.Q4_K, zb.Q6_K], ids=["q4_k", "q6_k"])
@pytest.mark.parametrize("act", ["f32", "bf16"])
@pytest.mark.parametrize("M,N,K", [(64, 16, 256), (300, 77, 1024), (1024, 256, 2048), (256, 300, 4096)])
def test_mul_mm(gpu, oracle, t, act, M, N, K):
    # D[col][row] = sum_k A[row][k] B[col][k], strided column-major B and D (src/compute/dmmv.zig:1045-1094)
    torch, ctx, dd = gpu
    g = synth.rng(301, t * 100 + M)
    w = synth.quant_matrix(g, t, M, K)
    Bm = synth.activations(g, N, K)
    stride_b, stride_d, b_off, d_off = K + 8, M + 4, 16, 8
    Bpad = np.zeros(b_off + N * stride_b, np.float32)
    for c in range(N):
        Bpad[b_off + c * stride_b: b_off + c * stride_b + K] = Bm[c]
    if act == "bf16":
        bits = synth.to_bf16_bits(Bpad)
        Bd = dev(torch, bits.view(np.int16))
        Bexact = synth.bf16_bits_to_f32(synth.to_bf16_bits(Bm))
    else:
        Bd = dev(torch, Bpad)
        Bexact = Bm
    D = out_with_canary(torch, d_off + N * stride_d)
    dd.recordMulMm(t, dev(torch, w), Bd, D, M, N, K, stride_b, stride_d, 0, b_off, d_off,
                   zb.BF16 if act == "bf16" else zb.F32)
    ctx.submit_and_wait()
    got = D[d_off:d_off + N * stride_d].cpu().numpy().reshape(N, stride_d)
    assert canary_intact(D, d_off + N * stride_d)
    assert np.all(got[:, M:] == 0.0), "padding between columns must stay untouched"
    exact = oracle.gemm_f64(w, t, M, K, Bexact)
    e = rel_l2(got[:, :M], exact)
    assert e <= TOL_BF16
    if e > TOL_F32:
        assert rel_l2(got[:, :M], oracle.gemm_f64(w, t, M, K, Bexact, round_bf16=True)) <= TOL_BF16_OPERANDS


@pytest.mark.parametrize("t", [zb.Q4_K, zb.Q6_K], ids=["q4_k", "q6_k"])
@pytest.mark.parametrize("M,N,K", [(2043, 2600, 1024), (1280, 4100, 512), (1026, 600, 2816)])
def test_mul_mm_cta_pairs(gpu, oracle, t, M, N, K):
    """Shapes with enough tiles that K is not split and an even number of 128-row tiles: the large-tile kernel runs
    as CTA pairs (one MMA of 256 rows per pair, each CTA fetching half of every activation box). Ragged last row
    tile, a last token tile that fills one accumulator only, strided B and D."""
    torch, ctx, dd = gpu
    g = synth.rng(304, t * 100 + M)
    w = synth.quant_matrix(g, t, M, K)
    Bm = synth.activations(g, N, K)
    stride_b, stride_d = K + 8, M + 5
    Bpad = np.zeros((N, stride_b), np.float32)
    Bpad[:, :K] = Bm
    bits = synth.to_bf16_bits(Bpad.reshape(-1))
    Bexact = synth.bf16_bits_to_f32(synth.to_bf16_bits(Bm.reshape(-1))).reshape(N, K)
    D = out_with_canary(torch, N * stride_d)
    dd.recordMulMm(t, dev(torch, w), dev(torch, bits.view(np.int16)), D, M, N, K, stride_b, stride_d, 0, 0, 0, zb.BF16)
    ctx.submit_and_wait()
    got = D[:N * stride_d].cpu().numpy().reshape(N, stride_d)
    assert canary_intact(D, N * stride_d)
    assert np.all(got[:, M:] == 0.0), "padding between columns must stay untouched"
    exact = oracle.gemm_f64(w, t, M, K, Bexact)
    assert rel_l2(got[:, :M], exact) <= TOL_BF16
    assert rel_l2(got[:, :M], oracle.gemm_f64(w, t, M, K, Bexact, round_bf16=True)) <= TOL_BF16_OPERANDS
    # every row tile against its own rows: a pair that swapped or dropped a half would pass no global norm
    for r0 in range(0, M, 128):
        assert rel_l2(got[:, r0:min(r0 + 128, M)], exact[:, r0:r0 + 128]) <= TOL_BF16
    for c0 in range(0, N, 128):
        assert rel_l2(got[c0:c0 + 128, :M], exact[c0:c0 + 128]) <= TOL_BF16


@pytest.mark.parametrize("M,N,K", [(2048, 1100, 6144), (512, 700, 2048)], ids=["flags", "zeroed"])
def test_mul_mm_cta_pairs_recorded(gpu, oracle, M, N, K):
    """The pair kernel inside a recording, replayed. Tiles split over pairs are summed through memory: with long
    ranges (24 tiles x 24 blocks over 74 pairs) behind per-tile flags that a memset node of the recording clears (a
    flag left up would let an adder run ahead of the stores it adds to, a flag left down would time out), with
    short ranges (4 tiles x 8 blocks over 8 pairs) by adding into D, which a memset node zeroes. Either way every
    replay has to give the product again."""
    torch, _, _ = gpu
    t = zb.Q4_K
    g = synth.rng(305, 1)
    w = synth.quant_matrix(g, t, M, K)
    Bm = synth.activations(g, N, K)
    bits = synth.to_bf16_bits(Bm.reshape(-1))
    Bexact = synth.bf16_bits_to_f32(bits).reshape(N, K)
    exact = oracle.gemm_f64(w, t, M, K, Bexact)
    stream = torch.cuda.Stream()   # a stream of its own: the default stream cannot be captured
    with torch.cuda.stream(stream):
        ctx = zb.Context(0, stream=stream.cuda_stream)
        dd = zb.DmmvDispatch(ctx)
        wd, bd = dev(torch, w), dev(torch, bits.view(np.int16))
        D = out_with_canary(torch, N * M)
        stream.synchronize()
        ctx.begin_record()
        dd.recordMulMm(t, wd, bd, D, M, N, K, K, M, 0, 0, 0, zb.BF16)
        rec = ctx.end_record()
        try:
            for _ in range(3):
                D[:N * M] = float("nan")
                ctx.replay(rec)
                ctx.submit_and_wait()
                got = D[:N * M].cpu().numpy().reshape(N, M)
                assert canary_intact(D, N * M)
                assert rel_l2(got, exact) <= TOL_BF16
        finally:
            ctx.free_recording(rec)


@pytest.mark.parametrize("M,N,K", [(64, 16, 64), (300, 77, 320), (200, 32, 2880), (256, 300, 2880),
                                   (1000, 700, 2880), (1152, 520, 448)])
def test_mul_mm_mxfp4_bf16(gpu, oracle, M, N, K):
    # MXFP4 weights dequantise exactly to bf16, so with bf16 activations the tensor-core product differs
    # from the exact one only by the f32 accumulation order (rows of 17-byte blocks: no alignment at all)
    torch, ctx, dd = gpu
    t = zb.MXFP4
    g = synth.rng(302, M + K)
    w = synth.quant_matrix(g, t, M, K)
    Bm = synth.activations(g, N, K)
    bits = synth.to_bf16_bits(Bm.reshape(-1))
    Bexact = synth.bf16_bits_to_f32(bits).reshape(N, K)
    D = out_with_canary(torch, N * M)
    dd.recordMulMm(t, dev(torch, w), dev(torch, bits.view(np.int16)), D, M, N, K, K, M, 0, 0, 0, zb.BF16)
    ctx.submit_and_wait()
    got = D[:N * M].cpu().numpy().reshape(N, M)
    assert canary_intact(D, N * M)
    assert rel_l2(got, oracle.gemm_f64(w, t, M, K, Bexact)) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 128, 512), (300, 200, 2880), (1024, 600, 2880), (130, 64, 160)])
def test_mul_mm_mxfp4_block_scaled(gpu, oracle, M, N, K):
    """MXFP4 weights as stored on the block-scaled tensor-core path (zc_mul_mm_block_scaled): the two FP8 terms add
    up to the bf16 activation exactly, so the product differs from the exact one by the f32 accumulation only.
    Row, token and K counts that are not multiples of the tile, a wide activation range inside a block, and the
    launch count (split + GEMM) that shows this path ran."""
    torch, ctx, dd = gpu
    t = zb.MXFP4
    g = synth.rng(303, M + K + N)
    w = synth.quant_matrix(g, t, M, K)
    Bm = synth.activations(g, N, K)
    Bm[:, ::7] *= np.float32(64.0)      # spread of magnitudes inside a 32-element block
    Bm[:, 3::11] *= np.float32(1.0 / 128.0)
    Bm[N // 2, :32] = 0.0               # an all-zero block
    bits = synth.to_bf16_bits(Bm.reshape(-1))
    Bexact = synth.bf16_bits_to_f32(bits).reshape(N, K)
    D = out_with_canary(torch, N * M)
    ws = torch.empty(dd.mulMmWorkspaceBytes(t, N, K), dtype=torch.uint8, device="cuda")
    assert ws.numel() > 0 and dd.mulMmWorkspaceBytes(zb.Q4_K, N, K) == 0
    n0 = ctx.launch_count
    dd.recordMulMmBlockScaled(t, dev(torch, w), dev(torch, bits.view(np.int16)), D, M, N, K, K, M, ws)
    ctx.submit_and_wait()
    assert ctx.launch_count - n0 == 2
    with pytest.raises(zb.InvalidArgument):   # a workspace that is too small
        dd.recordMulMmBlockScaled(t, dev(torch, w), dev(torch, bits.view(np.int16)), D, M, N, K, K, M, ws[:1024])
    with pytest.raises(zb.UnsupportedQuantType):
        dd.recordMulMmBlockScaled(zb.Q4_K, dev(torch, w), dev(torch, bits.view(np.int16)), D, M, N, K, K, M, ws)
    got = D[:N * M].cpu().numpy().reshape(N, M)
    assert canary_intact(D, N * M)
    assert rel_l2(got, oracle.gemm_f64(w, t, M, K, Bexact)) <= 1e-5


def test_mul_mm_errors(gpu):
    torch, ctx, dd = gpu
    w = torch.zeros(144 * 8, dtype=torch.uint8, device="cuda")
    b = torch.zeros(4 * 256, device="cuda")
    d = torch.zeros(4 * 8, device="cuda")
    with pytest.raises(zb.InvalidArgument):  # K misaligned (src/compute/dmmv.zig:1065)
        dd.recordMulMmQ4K(w, b, d, 8, 4, 200, 256, 8)
    with pytest.raises(zb.InvalidArgument):  # N == 0 (src/compute/dmmv.zig:1066)
        dd.recordMulMmQ4K(w, b, d, 8, 0, 256, 256, 8)
    with pytest.raises(zb.UnsupportedQuantType):
        dd.recordMulMm(11, w, b, d, 8, 4, 256, 256, 8)
    dd.recordMulMmQ4K(w, b, d, 8, 4, 256, 256, 8)
    ctx.submit_and_wait()
