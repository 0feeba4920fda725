"""NVFP4 weights as lex reads them from an Ollama-store safetensors blob
(crates/lex-rt/src/qwen.rs:217-250; scripts/qwen_nvfp4.py:57-92): three entries per matrix,

    name               U32 [rows, cols/8]   8 codes per little-endian word, value k in bits 4k..4k+3
    name.scale         U8  [rows, cols/16]  E4M3 bytes
    name.global_scale  F32 [1]              one scale for the tensor, spread over its rows

which are exactly (wq, ws, wg) of `gemm_fp4`: a little-endian word of 8 codes is 4 bytes with the even
column in the low nibble, so the codes need no repacking; the scalar becomes a per-row vector.
Only the blob format is handled here (8-byte header length, JSON header, data); the Ollama manifest that
maps a model name to blobs is not.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


def _read_blob(path):
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    head = json.loads(raw[8:8 + hlen])
    return head, memoryview(raw)[8 + hlen:]


def tensor_names(path) -> list[str]:
    head, _ = _read_blob(path)
    return [k for k in head if k != "__metadata__"]


def read_nvfp4(path, name: str):
    """(wq u8[rows, cols/2], ws u8[rows, cols/16], wg f32[rows]) of matrix `name`."""
    head, data = _read_blob(path)

    def part(key, dtype):
        if key not in head:
            raise KeyError(f"{key}: missing (is this weight NVFP4?)")
        e = head[key]
        lo, hi = e["data_offsets"]
        if hi > len(data):
            raise ValueError(f"{key}: data runs past the blob")
        if e["dtype"] != dtype:
            raise ValueError(f"{key}: dtype {e['dtype']}, expected {dtype}")
        return e, data[lo:hi]

    ce, codes = part(name, "U32")
    if len(ce["shape"]) != 2:
        raise ValueError(f"{name}: expected a matrix, got {ce['shape']}")
    rows, words = ce["shape"]
    se, scales = part(name + ".scale", "U8")
    _, gs = part(name + ".global_scale", "F32")
    if len(gs) < 4:
        raise ValueError("global scale is not four bytes")
    cols = words * 8
    if list(se["shape"]) != [rows, cols // 16]:
        raise ValueError(f"{name}.scale: shape {se['shape']} does not fit {rows} x {cols}")
    wq = np.frombuffer(codes, dtype=np.uint8).reshape(rows, cols // 2).copy()
    ws = np.frombuffer(scales, dtype=np.uint8).reshape(rows, cols // 16).copy()
    wg = np.full(rows, np.frombuffer(gs[:4], dtype="<f4")[0], dtype=np.float32)   # one per row (qwen.rs:248)
    return wq, ws, wg


def write_nvfp4(path, tensors: dict) -> None:
    """Write {name: (wq, ws, global_scale)} in the same blob format (for tests and synthetic checkpoints)."""
    head, chunks, off = {}, [], 0

    def add(key, dtype, shape, payload: bytes):
        nonlocal off
        head[key] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(payload)]}
        chunks.append(payload)
        off += len(payload)

    for name, (wq, ws, gs) in tensors.items():
        rows, half = wq.shape
        if half % 4:
            raise ValueError("cols must be a multiple of 8")
        add(name, "U32", (rows, half // 4), np.ascontiguousarray(wq, dtype=np.uint8).tobytes())
        add(name + ".scale", "U8", ws.shape, np.ascontiguousarray(ws, dtype=np.uint8).tobytes())
        add(name + ".global_scale", "F32", (1,), np.float32(gs).astype("<f4").tobytes())
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    Path(path).write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(chunks))
