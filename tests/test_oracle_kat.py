"""Known-answer tests that pin the CPU oracle to the reference's own unit tests.

Each test restates one test of the reference project (cited by path:lines):
the same bytes in, the same expected numbers out.
"""
import struct

import numpy as np

from oracle import oracle as o

F32, F16, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, MXFP4 = 0, 1, 6, 7, 8, 12, 13, 14, 39


def f16(v: float) -> bytes:
    return np.array([v], dtype=np.float16).tobytes()


def test_get_scale_min_k4_low():  # src/compute/forward.zig:11590-11599
    s = [0] * 12
    s[0], s[4] = 0xFF, 0xC5
    assert o.get_scale_min_k4(0, s) == (63, 5)


def test_get_scale_min_k4_high():  # src/compute/forward.zig:11601-11614
    s = [0] * 12
    s[0], s[4], s[8] = 0xC0, 0x80, 0x72
    assert o.get_scale_min_k4(4, s) == (50, 39)


def test_dequant_q4k_pairing():  # src/compute/forward.zig:11465-11497
    b = bytearray(144)
    b[0:2] = f16(1.0)
    b[4], b[5] = 1, 2
    b[16], b[17] = 0x53, 0x97
    out = o.dequant_row(np.frombuffer(bytes(b), np.uint8), 0, 256, Q4_K)
    assert out[0] == 3.0 and out[1] == 7.0 and out[32] == 10.0 and out[33] == 18.0


def test_dequant_q5k_halves():  # src/compute/forward.zig:11499-11527
    b = bytearray(176)
    b[0:2] = f16(1.0)
    b[4], b[5] = 1, 1
    b[48] = 0x3A
    out = o.dequant_row(np.frombuffer(bytes(b), np.uint8), 0, 256, Q5_K)
    assert out[0] == 10.0 and out[32] == 3.0


def test_q5k_dot_3010():  # src/compute/forward_metal.zig:11293-11331
    b = bytearray(176)
    b[0:2] = f16(1.0)
    b[4], b[5] = 1, 1
    b[48] = 0x3A
    x = np.zeros(256, np.float32)
    x[0], x[1], x[32] = 1.0, 100.0, 1000.0
    raw = np.frombuffer(bytes(b), np.uint8)
    row = o.dequant_row(raw, 0, 256, Q5_K)
    assert row[0] == 10.0 and row[1] == 0.0 and row[32] == 3.0
    assert o.dmmv_f32seq(raw, Q5_K, 1, 256, x)[0] == 3010.0


def test_dequant_q8_0():  # src/compute/forward.zig:11529-11553
    b = bytearray(34)
    b[0:2] = f16(0.5)
    b[2:6] = struct.pack("4b", 1, -1, 127, -128)
    out = o.dequant_row(np.frombuffer(bytes(b), np.uint8), 0, 32, Q8_0)
    assert list(out[:4]) == [0.5, -0.5, 63.5, -64.0] and out[6] == 0.0


def test_dequant_f16_f32():  # src/compute/forward.zig:11555-11584, 11762-11777
    raw = np.array([1.5, -3.25, 0.0, 42.0], np.float16).view(np.uint8)
    assert list(o.dequant_row(raw, 0, 4, F16)) == [1.5, -3.25, 0.0, 42.0]
    raw = np.array([1.0, -2.0, 3.14, 0.0], np.float32).view(np.uint8)
    assert list(o.dequant_row(raw, 0, 4, F32)) == [1.0, -2.0, np.float32(3.14), 0.0]
    raw = np.array([1.0, -0.5, 0.25, 100.0], np.float16).view(np.uint8)
    assert list(o.dequant_row(raw, 0, 4, F16)) == [1.0, -0.5, 0.25, 100.0]


def test_dequant_q5_0_qh_bit16():  # src/compute/forward_metal.zig:11234-11249
    b = bytearray(22)
    b[0:2] = f16(1.0)
    b[2:6] = struct.pack("<I", 1 << 16)
    out = o.dequant_row(np.frombuffer(bytes(b), np.uint8), 0, 32, Q5_0)
    assert out[0] == -16.0 and out[16] == 0.0


def test_dequant_q5_1_qh_bit16():  # src/compute/forward_metal.zig:11251-11269
    b = bytearray(24)
    b[0:2] = f16(1.0)
    b[2:4] = f16(0.0)
    b[4:8] = struct.pack("<I", 1 << 16)
    out = o.dequant_row(np.frombuffer(bytes(b), np.uint8), 0, 32, Q5_1)
    assert out[0] == 0.0 and out[16] == 16.0


def test_q5_1_factored_dot():  # src/regression_tests.zig:605-629 (d=0.5, qh=0x0000FFFF, qs=0x53)
    b = bytearray(24)
    b[0:2] = f16(0.5)
    b[2:4] = f16(-8.0)
    b[4:8] = struct.pack("<I", 0x0000FFFF)
    b[8:24] = bytes([0x53] * 16)
    out = o.dequant_row(np.frombuffer(bytes(b), np.uint8), 0, 32, Q5_1)
    # low nibble 3 | bit 16 -> 19 -> 0.5*19 - 8 = 1.5 ; high nibble 5, bit 0 -> 0.5*5 - 8 = -5.5
    assert np.all(out[:16] == 1.5) and np.all(out[16:] == -5.5)


def test_mxfp4_dot_48():  # src/compute/forward_metal.zig:14238-14303
    rows = bytearray()
    for _ in range(4):
        rows += bytes([127]) + bytes([0x42] * 16)
    raw = np.frombuffer(bytes(rows), np.uint8)
    y = o.dmmv_f32seq(raw, MXFP4, 4, 32, np.ones(32, np.float32))
    assert list(y) == [48.0] * 4
    row = o.dequant_row(raw, 0, 32, MXFP4)
    assert np.all(row[:16] == 1.0) and np.all(row[16:] == 2.0)


def test_mxfp4_lut_and_e0():  # src/compute/forward.zig:441-459
    lut = [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    qs = bytes((2 * i) | ((2 * i + 1) << 4) for i in range(8)) + bytes(8)
    raw = np.frombuffer(bytes([128]) + qs, np.uint8)  # e = 128 -> scale 2
    row = o.dequant_row(raw, 0, 32, MXFP4)
    for i in range(8):
        assert row[i] == 2 * lut[2 * i] and row[16 + i] == 2 * lut[2 * i + 1]
    raw0 = np.frombuffer(bytes([0]) + bytes([0x22] * 16), np.uint8)  # e = 0 -> 2^-127
    assert o.dequant_row(raw0, 0, 32, MXFP4)[0] == np.float32(2.0 ** -127)


def test_expert_slice_bytes():  # src/compute/forward.zig:11409-11423, 11737-11756; forward_metal.zig:11219-11222
    assert o.expert_slice_bytes(Q4_K, 512, 2048) == 589_824
    assert o.expert_slice_bytes(Q5_K, 2048, 512) == 720_896
    assert o.expert_slice_bytes(Q6_K, 256, 2048) == 430_080
    assert o.expert_slice_bytes(Q8_0, 2048, 2048) == 4_456_448
    assert o.expert_slice_bytes(F16, 512, 2048) == 2_097_152
    assert o.expert_slice_bytes(Q4_K, 1024, 2048) == 1024 * 8 * 144


def test_block_geometry_and_size_bytes():  # src/model/gguf.zig:545-576
    assert (o.block_size(Q4_K), o.bytes_per_block(Q4_K)) == (256, 144)
    assert (o.block_size(Q8_0), o.bytes_per_block(Q8_0)) == (32, 34)
    assert (o.block_size(F32), o.bytes_per_block(F32)) == (1, 4)
    assert (o.block_size(MXFP4), o.bytes_per_block(MXFP4)) == (32, 17)
    assert o.tensor_size_bytes(Q4_K, 4096 * 4096) == 9_437_184
    assert o.tensor_size_bytes(F32, 1024) == 4096


def test_bytes_model():  # src/bench_hot_decode.zig:785-787
    assert o.dmmv_bytes_model(Q8_0, 256, 2048) == 566_272


def test_topk_softmax_basic():  # src/compute/forward.zig:11392-11407
    ids, w = o.topk_softmax([1.0, 3.0, 0.5, 2.0, 4.0, 1.5, 0.1, 0.2], 3)
    assert list(ids) == [4, 1, 3]
    assert abs(w.sum() - 1.0) < 0.01 and w[0] > w[1] > w[2]


def test_topk_softmax_edges():  # src/compute/forward.zig:11620-11676
    ids, w = o.topk_softmax([1.0, 1.0, 1.0, 1.0], 2)
    assert list(ids) == [0, 1] and abs(w[0] - 0.5) < 0.01 and abs(w[1] - 0.5) < 0.01
    ids, w = o.topk_softmax([-1.0, 5.0, 2.0], 1)
    assert ids[0] == 1 and abs(w[0] - 1.0) < 1e-3
    ids, w = o.topk_softmax([100.0, 0.0, -100.0], 2)
    assert list(ids) == [0, 1] and w[0] > 0.99 and abs(w.sum() - 1.0) < 1e-3


def _selected_softmax(logits, ids):
    sel = np.array([logits[i] for i in ids], np.float32)
    e = np.exp(sel - sel.max())
    return e / e.sum()


def test_topk_rules_match_selected_softmax():  # src/compute/forward.zig:11630-11653, 11678-11710
    lg = [-2.0, 1.5, 0.25, 4.0, -0.5, 3.0, 2.5, -1.0]
    ids, w = o.topk_softmax(lg, 4)
    assert np.allclose(w, _selected_softmax(lg, ids), atol=1e-6)
    lg = [-3.0, 1.5, 0.25, 4.0, -0.5, 3.0, 2.5, -1.0]
    ids, w = o.topk_softmax_weight(lg, 4)
    assert list(ids) == [3, 5, 6, 1]
    assert np.allclose(w, _selected_softmax(lg, ids), atol=1e-6)
    ids, w = o.topk_softmax_weight([-9.0, -2.0, -5.0], 1)
    assert ids[0] == 1 and abs(w[0] - 1.0) < 1e-3


def test_silu():  # src/compute/forward.zig:11852-11862
    out = o.swiglu([0.0, 1.0, -1.0, 10.0], [1.0, 1.0, 1.0, 1.0])
    assert abs(out[0]) < 1e-7 and abs(out[1] - 0.7310586) < 1e-5 and abs(out[2] + 0.2689414) < 1e-5
    assert abs(out[3] - 10.0) < 1e-3


def test_swiglu_oai_formula():  # src/compute/forward.zig:607-616 (no known answer in the reference)
    g = np.array([-3.0, 0.5, 9.0], np.float32)
    u = np.array([-9.0, 0.25, 8.0], np.float32)
    gc, uc = np.minimum(g, 7), np.clip(u, -7, 7)
    want = gc / (1 + np.exp(1.702 * -gc)) * (uc + 1)
    assert np.allclose(o.swiglu(g, u, oai=True), want, rtol=1e-6)


def test_q6k_three_way_formula():
    """Q6_K has no known answer in the reference; check the oracle against an
    independent numpy restatement of the rule (src/compute/forward.zig:276-325)."""
    g = np.random.default_rng(7)
    raw = g.integers(0, 256, 210 * 3, dtype=np.uint8)
    for blk in range(3):
        raw[210 * blk + 208:210 * blk + 210] = np.frombuffer(f16(0.01 * (blk + 1)), np.uint8)
    got = o.dequant_row(raw, 0, 768, Q6_K)
    for blk in range(3):
        b = raw[210 * blk:210 * (blk + 1)]
        d = np.float32(np.frombuffer(b[208:210].tobytes(), np.float16)[0])
        sc = b[192:208].view(np.int8).astype(np.float32)
        for i in range(256):
            half, r = divmod(i, 128)
            quarter, l = divmod(r, 32)
            ql = b[64 * half + l + (32 if quarter & 1 else 0)]
            nib = (ql >> 4) if quarter & 2 else (ql & 0xF)
            q = int(nib | (((b[128 + 32 * half + l] >> (2 * quarter)) & 3) << 4)) - 32
            want = np.float32(np.float32(d * sc[8 * half + l // 16 + 2 * quarter]) * np.float32(q))
            assert got[256 * blk + i] == want


def test_shader_order_matches_f64(oracle):
    """The timed CPU baseline (shader lane order) agrees with the f64 product."""
    from zinc_b200 import synth

    for t, K in ((Q4_K, 1024), (Q5_K, 512), (Q6_K, 1024), (Q8_0, 256), (MXFP4, 2880)):
        g = synth.rng(0, t)
        w = synth.quant_matrix(g, t, 9, K)
        x = synth.activations(g, K)
        a = oracle.dmmv_shader_order(w, t, 9, K, x).astype(np.float64)
        b = oracle.dmmv_f64(w, t, 9, K, x)
        assert np.linalg.norm(a - b) / np.linalg.norm(b) < 1e-5
