"""Shared helpers of the GPU parity tests."""
import numpy as np

CANARY = 0xA5


def rel_l2(got, want) -> float:
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (den if den > 0 else 1.0))


def dev(torch, arr: np.ndarray):
    """Upload a numpy array to cuda:0 (as its raw dtype; uint8 for weight bytes)."""
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def dev_padded(torch, arr: np.ndarray, front: int = 0, back: int = 64, fill: int = CANARY):
    """Upload bytes with poisoned padding either side; returns (tensor, front_offset)."""
    raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
    buf = np.full(front + raw.size + back, fill, dtype=np.uint8)
    buf[front:front + raw.size] = raw
    return torch.from_numpy(buf).cuda(), front


def out_with_canary(torch, n_floats: int, back: int = 16, init: float = 0.0):
    """f32 output buffer followed by canary words that a correct kernel never writes."""
    t = torch.full((n_floats + back,), float("nan"), dtype=torch.float32, device="cuda")
    t[:n_floats] = init
    return t


def canary_intact(t, n_floats: int) -> bool:
    return bool(t[n_floats:].isnan().all().item())


def oracle_moe_decode_layer(o, x, router, wg, wu, wd, shape, ffn, router_bias=None, bg=None, bu=None, bd=None,
                            sg=None, su=None, sd=None):
    """One MoE layer's contribution to the hidden vector, composed from the oracle's primitives in the order
    of the reference's MoE blocks (src/compute/forward.zig:6139-6545 GPU-routed, 6712-6930 CPU-routed):
    router matvec (+ bias) -> top-k -> per selected expert gate / up (+ biases) -> activation -> down (+ bias)
    -> weighted sum -> shared expert. `ffn` is the expert FFN width the weight tensors hold. Returns
    (hidden contribution f64 [hidden], expert ids)."""
    from zinc_b200 import synth
    s = shape
    H, E, k, F = s.hidden, s.n_experts, s.top_k, ffn
    logits = (np.asarray(router, np.float64).reshape(E, H) @ x.astype(np.float64)).astype(np.float32)
    if router_bias is not None:
        logits = logits + np.asarray(router_bias, np.float32)
    ids, wts = (o.topk_softmax if s.rule == 0 else o.topk_softmax_weight)(logits, k)
    es_gu = F * (H // synth.BLOCK[s.t_gate_up][0]) * synth.BLOCK[s.t_gate_up][1]
    es_d = H * (F // synth.BLOCK[s.t_down][0]) * synth.BLOCK[s.t_down][1]
    xs = np.repeat(x[None, :], k, axis=0)
    gate = o.moe_dmmv_f64(wg, s.t_gate_up, F, H, es_gu, ids, H, xs).astype(np.float32)
    up = o.moe_dmmv_f64(wu, s.t_gate_up, F, H, es_gu, ids, H, xs).astype(np.float32)
    if bg is not None:
        gate = gate + np.asarray(bg, np.float32).reshape(E, F)[ids]
    if bu is not None:
        up = up + np.asarray(bu, np.float32).reshape(E, F)[ids]
    act = o.swiglu(gate.reshape(-1), up.reshape(-1), oai=s.oai).reshape(k, F)
    down = o.moe_dmmv_f64(wd, s.t_down, H, F, es_d, ids, F, act)
    if bd is not None:
        down = down + np.asarray(bd, np.float64).reshape(E, H)[ids]
    out = (wts.astype(np.float64)[:, None] * down).sum(0)
    if sg is not None:
        g1 = o.dmmv_f64(sg, s.t_gate_up, F, H, x).astype(np.float32)
        u1 = o.dmmv_f64(su, s.t_gate_up, F, H, x).astype(np.float32)
        out = out + o.dmmv_f64(sd, s.t_down, H, F, o.swiglu(g1, u1, oai=s.oai))
    return out, ids
