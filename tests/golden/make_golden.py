"""Writes tests/golden/hot_path_small.npz: small seeded inputs of the hot path with the outputs of the
CPU oracle (oracle/zinc_oracle.cpp), which restates the reference's CPU math
(src/compute/forward.zig:242-465 dequantRow, 496-571 topKSoftmax*, 607-616 SiLU).

The reference is a Zig program and cannot be run here; its own known answers are transcribed in
tests/test_oracle_kat.py and pin the oracle. This file pins the oracle's outputs on wider seeded
inputs so that a later change of the oracle or of the generators cannot move the parity target
silently.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as zo  # noqa: E402
from zinc_b200 import synth  # noqa: E402
from zinc_b200 import _lib as zb  # noqa: E402

TYPES = [zb.Q4_K, zb.Q5_K, zb.Q6_K, zb.Q8_0, zb.MXFP4, zb.Q5_0, zb.Q5_1, zb.F16, zb.F32]
M, K = 9, 512


def main():
    out = {}
    for t in TYPES:
        g = synth.rng(200, t)
        w = synth.quant_matrix(g, t, M, K)
        x = synth.activations(g, K)
        name = zb.TYPE_NAMES[t]
        out[f"{name}_w"] = w.reshape(-1)
        out[f"{name}_x"] = x
        out[f"{name}_dequant"] = zo.dequant_rows(w, M, K, t)   # f32, the bit-exact target
        out[f"{name}_y"] = zo.dmmv_f64(w, t, M, K, x)          # f64 dot of the dequantised rows
    g = synth.rng(201, 0)
    logits = synth.activations(g, 128)
    for k in (1, 4, 8):
        ids, wts = zo.topk_softmax(logits, k)
        out[f"route_all_k{k}_ids"], out[f"route_all_k{k}_w"] = ids, wts
        ids, wts = zo.topk_softmax_weight(logits, k)
        out[f"route_topk_k{k}_ids"], out[f"route_topk_k{k}_w"] = ids, wts
    out["route_logits"] = logits
    gate, up = synth.activations(g, 300) * np.float32(3), synth.activations(g, 300) * np.float32(3)
    out["act_gate"], out["act_up"] = gate, up
    out["act_swiglu"] = zo.swiglu(gate, up)
    out["act_swiglu_oai"] = zo.swiglu(gate, up, oai=True)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hot_path_small.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
