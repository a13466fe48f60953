"""Seeded synthetic GGUF-block tensors and activations.

These stand in for real model weights: the value distributions are the ones
the benchmark configurations name (f16 d, dmin ~ U[1e-3, 2e-2]; 6-bit scales
and mins ~ U{0..63}; uniform quant bytes; Q6_K int8 scales uniform; MXFP4
E8M0 exponents 127 + U{-8..0}). f16 fields are always finite.

`numpy` generators give bit-reproducible host arrays for parity tests;
`torch_*` generators fill large tensors directly on the device for the
benchmark (same distributions, torch's generator).
"""
from __future__ import annotations

import numpy as np

from ._lib import F16, F32, MXFP4, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0

BLOCK = {F32: (1, 4), F16: (1, 2), Q5_0: (32, 22), Q5_1: (32, 24), Q8_0: (32, 34),
         Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), MXFP4: (32, 17)}

SEED_BASE = 0x5EED0000


def rng(config_index: int, stream: int = 0) -> np.random.Generator:
    """One generator per (benchmark configuration, tensor)."""
    return np.random.Generator(np.random.Philox(key=SEED_BASE + config_index, counter=[stream, 0, 0, 0]))


def _f16_bytes(g: np.random.Generator, n: int, lo=1e-3, hi=2e-2) -> np.ndarray:
    return g.uniform(lo, hi, size=n).astype(np.float16).view(np.uint8).reshape(n, 2)


def _pack_k4_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Pack 8 six-bit scales and 8 six-bit mins per block into the 12-byte K-quant field."""
    n = sc.shape[0]
    out = np.zeros((n, 12), dtype=np.uint8)
    for j in range(4):
        out[:, j] = (sc[:, j] & 63) | ((sc[:, j + 4] >> 4) << 6)
        out[:, j + 4] = (mn[:, j] & 63) | ((mn[:, j + 4] >> 4) << 6)
        out[:, j + 8] = (sc[:, j + 4] & 0xF) | ((mn[:, j + 4] & 0xF) << 4)
    return out


def quant_blocks(g: np.random.Generator, qtype: int, n_blocks: int) -> np.ndarray:
    """n_blocks random blocks of the given type as a [n_blocks, bytes_per_block] uint8 array."""
    bpb = BLOCK[qtype][1]
    if qtype == F32:
        return g.standard_normal(n_blocks).astype(np.float32).view(np.uint8).reshape(n_blocks, 4)
    if qtype == F16:
        return g.standard_normal(n_blocks).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    b = g.integers(0, 256, size=(n_blocks, bpb), dtype=np.uint8)
    if qtype in (Q4_K, Q5_K):
        b[:, 0:2] = _f16_bytes(g, n_blocks)
        b[:, 2:4] = _f16_bytes(g, n_blocks)
        sc = g.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
        mn = g.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
        b[:, 4:16] = _pack_k4_scales(sc, mn)
    elif qtype == Q6_K:
        b[:, 208:210] = _f16_bytes(g, n_blocks)
    elif qtype in (Q8_0, Q5_0):
        b[:, 0:2] = _f16_bytes(g, n_blocks)
        if qtype == Q8_0:  # qs ~ U{-127..127}
            q = g.integers(-127, 128, size=(n_blocks, 32), dtype=np.int8)
            b[:, 2:34] = q.view(np.uint8)
    elif qtype == Q5_1:
        b[:, 0:2] = _f16_bytes(g, n_blocks)
        b[:, 2:4] = g.uniform(-2e-2, 2e-2, size=n_blocks).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    elif qtype == MXFP4:
        b[:, 0] = (127 - g.integers(0, 9, size=n_blocks)).astype(np.uint8)
    return b


def quant_matrix(g: np.random.Generator, qtype: int, M: int, K: int) -> np.ndarray:
    """Raw bytes of an M x K weight matrix, rows of K/block_size blocks."""
    bs = BLOCK[qtype][0]
    assert K % bs == 0
    return quant_blocks(g, qtype, M * (K // bs)).reshape(-1)


def activations(g: np.random.Generator, *shape: int) -> np.ndarray:
    return g.standard_normal(size=shape).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16, returned as uint16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


# ---- arithmetic-pattern fixtures of the reference's kernel tests -------------------------------
def pattern_q5k(M=257, K=512) -> tuple[np.ndarray, np.ndarray]:
    """Weight bytes and input of the Q5_K many-rows test (src/compute/forward_metal.zig:11419-11464)."""
    bpr = K // 256
    w = np.zeros((M, bpr, 176), dtype=np.uint8)
    for row in range(M):
        for blk in range(bpr):
            b = w[row, blk]
            b[0:2] = np.array([0.03125 * (1 + (row % 5) + blk)], dtype=np.float16).view(np.uint8)
            b[2:4] = np.array([0.015625 * (1 + ((row + blk) % 7))], dtype=np.float16).view(np.uint8)
            i = np.arange(12)
            b[4:16] = (row * 9 + blk * 5 + i * 3) & 0xFF
            i = np.arange(32)
            b[16:48] = (row * 7 + blk * 11 + i * 5) & 0xFF
            i = np.arange(128)
            b[48:176] = (row * 13 + blk * 17 + i * 7) & 0xFF
    i = np.arange(K)
    x = (0.125 * (((i * 19 + 5) % 21) - 10)).astype(np.float32)
    return w.reshape(-1), x


def pattern_q6k(M=257, K=512) -> tuple[np.ndarray, np.ndarray]:
    """Weight bytes and input of the Q6_K many-rows test (src/compute/forward_metal.zig:11508-11546)."""
    bpr = K // 256
    w = np.zeros((M, bpr, 210), dtype=np.uint8)
    for row in range(M):
        for blk in range(bpr):
            b = w[row, blk]
            i = np.arange(192)
            b[0:192] = (row * 23 + blk * 17 + i * 7) & 0xFF
            i = np.arange(16)
            b[192:208] = (row * 29 + blk * 19 + i * 5) & 0xFF
            b[208:210] = np.array([0.03125 * (1 + (row % 5) + blk)], dtype=np.float16).view(np.uint8)
    i = np.arange(K)
    x = (0.125 * (((i * 17 + 9) % 25) - 12)).astype(np.float32)
    return w.reshape(-1), x


def pattern_q4k_moe(M=65, K=512, n_experts=3, n_used=2) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Stacked Q4_K experts, per-slot inputs and routing ids of the MoE test
    (src/compute/forward_metal.zig:11590-11646)."""
    bpr = K // 256
    w = np.zeros((n_experts, M, bpr, 144), dtype=np.uint8)
    for e in range(n_experts):
        for row in range(M):
            for blk in range(bpr):
                b = w[e, row, blk]
                b[0:2] = np.array([0.03125 * (1 + e + (row % 5) + blk)], dtype=np.float16).view(np.uint8)
                b[2:4] = np.array([0.015625 * (1 + ((e + row + blk) % 7))], dtype=np.float16).view(np.uint8)
                i = np.arange(12)
                b[4:16] = (e * 31 + row * 9 + blk * 5 + i * 3) & 0xFF
                i = np.arange(128)
                lo = (e * 19 + row * 13 + blk * 17 + i * 7) & 0x0F
                hi = (e * 11 + row * 5 + blk * 3 + i * 9) & 0x0F
                b[16:144] = lo | (hi << 4)
    x = np.zeros((n_used, K), dtype=np.float32)
    i = np.arange(K)
    for slot in range(n_used):
        x[slot] = 0.125 * (((slot * 23 + i * 19 + 5) % 21) - 10)
    routing = np.array([2, 0], dtype=np.uint32)[:n_used]
    return w.reshape(-1), x, routing


# ---- device-side generators (benchmark-sized tensors) ---------------------------------------------
def torch_quant_matrix(qtype: int, M: int, K: int, device, seed: int):
    """Random weight matrix generated on the device: uint8 tensor of M * row_bytes bytes."""
    import torch

    bs, bpb = BLOCK[qtype]
    n = M * (K // bs)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    b = torch.randint(0, 256, (n, bpb), dtype=torch.uint8, device=device, generator=gen)

    def f16_field(lo, hi):
        v = torch.rand(n, device=device, generator=gen) * (hi - lo) + lo
        return v.to(torch.float16).view(torch.uint8).reshape(n, 2)

    if qtype in (Q4_K, Q5_K):
        b[:, 0:2] = f16_field(1e-3, 2e-2)
        b[:, 2:4] = f16_field(1e-3, 2e-2)  # the 12 scale bytes stay uniform: every 6-bit field is U{0..63}
    elif qtype == Q6_K:
        b[:, 208:210] = f16_field(1e-3, 2e-2)
    elif qtype in (Q8_0, Q5_0):
        b[:, 0:2] = f16_field(1e-3, 2e-2)
    elif qtype == Q5_1:
        b[:, 0:2] = f16_field(1e-3, 2e-2)
        b[:, 2:4] = f16_field(-2e-2, 2e-2)
    elif qtype == MXFP4:
        b[:, 0] = (127 - torch.randint(0, 9, (n,), device=device, generator=gen)).to(torch.uint8)
    elif qtype in (F32, F16):
        raise ValueError("use torch.randn for plain float tensors")
    return b.reshape(-1)
