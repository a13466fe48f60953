"""Tensor-parallel sharding of GGUF weight tensors (host side, numpy only).

The reference runs on one GPU; these helpers define how its tensors are cut for N GPUs:

* row shard: rank r owns output rows [r*M/N, (r+1)*M/N) -- a contiguous byte range of the tensor,
  because a row is `K / block_size` whole blocks (src/model/gguf.zig:222-229 sizeBytes). The
  outputs of the ranks are concatenated (all-gather).
* K shard: rank r owns blocks [r*nb/N, (r+1)*nb/N) of every row (nb = K / block_size). The blocks
  of one row are contiguous along K, so the shard is a strided gather that is re-laid out as its
  own dense [M][K/N] tensor. The outputs of the ranks are summed (all-reduce).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .dispatch import block_size, bytes_per_block


def _as_rows(raw, qtype: int, M: int, K: int) -> np.ndarray:
    bs, bpb = block_size(qtype), bytes_per_block(qtype)
    if K % bs:
        raise ValueError(f"K={K} is not a multiple of the block size {bs}")
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    need = M * (K // bs) * bpb
    if raw.size < need:
        raise ValueError(f"tensor holds {raw.size} bytes, {need} needed for {M} x {K}")
    return raw[:need].reshape(M, K // bs, bpb)


def row_range(M: int, rank: int, world: int) -> tuple[int, int]:
    if M % world:
        raise ValueError(f"M={M} does not divide over {world} ranks")
    n = M // world
    return rank * n, (rank + 1) * n


def row_shard(raw, qtype: int, M: int, K: int, rank: int, world: int) -> np.ndarray:
    """Bytes of rank's rows: a view of a contiguous range, no copy."""
    r0, r1 = row_range(M, rank, world)
    return _as_rows(raw, qtype, M, K)[r0:r1].reshape(-1)


def k_range(qtype: int, K: int, rank: int, world: int) -> tuple[int, int]:
    """Element range [k0, k1) of rank's K shard; whole blocks only."""
    nb = K // block_size(qtype)
    if K % block_size(qtype) or nb % world:
        raise ValueError(f"K={K}: {nb} blocks of type {qtype} do not divide over {world} ranks")
    n = nb // world
    return rank * n * block_size(qtype), (rank + 1) * n * block_size(qtype)


def k_shard(raw, qtype: int, M: int, K: int, rank: int, world: int) -> np.ndarray:
    """Rank's K shard re-laid out as a dense [M][K/world] tensor (a copy)."""
    k0, k1 = k_range(qtype, K, rank, world)
    bs = block_size(qtype)
    return np.ascontiguousarray(_as_rows(raw, qtype, M, K)[:, k0 // bs:k1 // bs]).reshape(-1)


@dataclass(frozen=True)
class MatShard:
    """One projection on one rank: local shape and where its input / output sit in the full vectors."""
    kind: str      # "row" or "k"
    M: int         # local rows
    K: int         # local columns
    y_begin: int   # first element of the full output this rank writes (row shard), 0 for a K shard
    x_begin: int   # first element of the full input this rank reads (K shard), 0 for a row shard


def plan(kind: str, M: int, K: int, qtype: int, rank: int, world: int) -> MatShard:
    if kind == "row":
        r0, r1 = row_range(M, rank, world)
        return MatShard("row", r1 - r0, K, r0, 0)
    if kind == "k":
        k0, k1 = k_range(qtype, K, rank, world)
        return MatShard("k", M, k1 - k0, 0, k0)
    raise ValueError(f"unknown shard kind {kind!r}")
