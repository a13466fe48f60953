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
