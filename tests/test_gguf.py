"""GGUF reader (include/zinc_gguf.hpp) against files written here with the container layout the
reference parses (src/model/gguf.zig:335-414): header, typed metadata, tensor table, aligned data."""
import os
import struct
import subprocess

import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "_build", "test_gguf")


def _build():
    from zinc_b200 import _lib

    _lib.lib()
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    libdir = os.path.dirname(_lib.SO_PATH)
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "test_gguf.cpp"), "-o", EXE, "-L", libdir, "-lzinc_b200",
                    "-Wl,-rpath," + libdir], check=True, capture_output=True, text=True)


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors, alignment=None, magic=0x46554747, truncate=None):
    """tensors: list of (name, dims, type id, raw bytes). Returns (data_offset, [tensor offsets])."""
    kv = [(_s("general.architecture") + struct.pack("<I", 8) + _s("qwen3")),
          (_s("test.block_count") + struct.pack("<Ii", 5, 36)),                 # int32 -> getU32
          (_s("test.rope_base") + struct.pack("<Id", 12, 1000000.0)),           # float64 -> getF32
          (_s("test.flag") + struct.pack("<IB", 0, 1)),                         # uint8 -> getBool
          (_s("test.list") + struct.pack("<IIQ", 9, 8, 3) + _s("a") + _s("bc") + _s("def"))]
    if alignment is not None:
        kv.append(_s("general.alignment") + struct.pack("<II", 4, alignment))
    al = alignment or 32
    head = struct.pack("<IIQQ", magic, 3, len(tensors), len(kv)) + b"".join(kv)
    offsets, off = [], 0
    table = b""
    for name, dims, t, raw in tensors:
        off = (off + al - 1) // al * al
        offsets.append(off)
        table += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        table += struct.pack("<IQ", t, off)
        off += len(raw)
    head += table
    data_offset = (len(head) + al - 1) // al * al
    blob = bytearray(head + b"\0" * (data_offset - len(head)))
    for (name, dims, t, raw), o in zip(tensors, offsets):
        blob += b"\0" * (data_offset + o - len(blob))
        blob += raw
    if truncate:
        blob = blob[:truncate]
    with open(path, "wb") as f:
        f.write(blob)
    return data_offset, offsets


def _tensors():
    g = synth.rng(500, 0)
    return [("blk.0.attn_q.weight", (512, 64), zb.Q4_K, synth.quant_matrix(g, zb.Q4_K, 64, 512).tobytes()),
            ("blk.0.ffn_down.weight", (2048, 6), zb.Q6_K, synth.quant_matrix(g, zb.Q6_K, 6, 2048).tobytes()),
            ("blk.0.ffn_gate_exps.weight", (64, 32, 4), zb.MXFP4, synth.quant_matrix(g, zb.MXFP4, 128, 64).tobytes()),
            ("output_norm.weight", (512,), zb.F32, np.arange(512, dtype=np.float32).tobytes())]


def _parse(path, *extra):
    _build()
    r = subprocess.run([EXE, path, *extra], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout.splitlines()


@pytest.mark.parametrize("alignment", [None, 64])
def test_parse_matches_what_was_written(tmp_path, alignment):
    ts = _tensors()
    path = str(tmp_path / "m.gguf")
    data_offset, offsets = write_gguf(path, ts, alignment)
    out = _parse(path)
    assert out[0] == f"version 3 tensors {len(ts)} data_offset {data_offset}"
    assert out[1:6] == ["arch qwen3", "block_count 36", "rope_base 1000000.0", "flag 1", "list 3"]
    for line, (name, dims, t, raw), o in zip(out[6:], ts, offsets):
        d = list(dims) + [1] * (3 - len(dims))
        want = (f"tensor {name} n_dims {len(dims)} dims {d[0]} {d[1]} {d[2]} type {t} offset {o} "
                f"bytes {len(raw)} sum {int(np.frombuffer(raw, np.uint8).sum(dtype=np.uint64))}")
        assert line == want


def test_errors(tmp_path):
    ts = _tensors()
    bad = str(tmp_path / "bad.gguf")
    write_gguf(bad, ts, magic=0x12345678)
    assert _parse(bad) == ["error InvalidMagic"]
    cut = str(tmp_path / "cut.gguf")
    write_gguf(cut, ts, truncate=60)
    assert _parse(cut) == ["error UnexpectedEof"]
    short = str(tmp_path / "short.gguf")
    data_offset, offsets = write_gguf(short, ts)
    with open(short, "r+b") as f:  # drop the last tensor's bytes: the table then points outside the file
        f.truncate(data_offset + offsets[-1] + 100)
    assert any(l.startswith("tensor output_norm.weight error InvalidTensor") for l in _parse(short))
    # dimensions whose product overflows 64 bits: refused while the table is read
    wrap = str(tmp_path / "wrap.gguf")
    write_gguf(wrap, [("w", [1 << 33, 1 << 33], 12, b"\0" * 144)] + ts)
    assert _parse(wrap)[0].startswith("error InvalidTensor")


@pytest.mark.gpu
def test_upload_round_trip(tmp_path):
    ts = _tensors()
    path = str(tmp_path / "m.gguf")
    write_gguf(path, ts)
    out = _parse(path, "--device")
    ups = [l for l in out if l.startswith("upload ")]
    assert len(ups) == len(ts) and all(l.endswith(" same") for l in ups)
    # 2-D tensors with an even row count were loaded as rank 1 of 2: half the bytes
    assert f"upload blk.0.attn_q.weight bytes {len(ts[0][3]) // 2} same" in ups
