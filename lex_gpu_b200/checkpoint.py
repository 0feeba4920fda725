"""NVFP4 weights as lex reads them from an Ollama-store safetensors blob
(crates/lex-rt/src/qwen.rs:217-250; scripts/qwen_nvfp4.py:57-92): three entries per matrix,

    name               U32 [rows, cols/8]   8 codes per little-endian word, value k in bits 4k..4k+3
    name.scale         U8  [rows, cols/16]  E4M3 bytes
    name.global_scale  F32 [1]              one scale for the tensor, spread over its rows

which are exactly (wq, ws, wg) of `gemm_fp4`: a little-endian word of 8 codes is 4 bytes with the even
column in the low nibble, so the codes need no repacking; the scalar becomes a per-row vector.
`read_nvfp4` / `write_nvfp4` handle one blob (8-byte header length, JSON header, data).  `Store` is the Ollama
store around the blobs (crates/lex-rt/src/qwen.rs:86-145): a manifest `manifests/registry.ollama.ai/library/
<name>/<tag>` whose named layers map tensor names to `blobs/<digest>` files, one tensor per blob.  A rank of an
n-sharded run reads only its own rows of each matrix (`rows=`, `Store.nvfp4_shard`): whole 128-row tiles as
lexb_shard_rows deals them, so that no rank ever holds the full matrix; `Store.gate_up_shard` reads a rank's
rows of gate and up and interleaves them for the fused gate/up launch.
"""
from __future__ import annotations

import hashlib
import json
import os
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


def _read_header(path):
    """The header of a blob and the file offset at which its data section starts, without reading the data."""
    with open(path, "rb") as f:
        first = f.read(8)
        if len(first) < 8:
            raise ValueError(f"{path}: too short for a header")
        (hlen,) = struct.unpack("<Q", first)
        head = f.read(hlen)
        if len(head) < hlen:
            raise ValueError(f"{path}: header runs past the blob")
    return json.loads(head), 8 + hlen


def read_nvfp4_rows(path, name: str, n0: int, n1: int):
    """Rows [n0, n1) of matrix `name`: only those bytes of the blob are read (a rank's slab of an n-sharded matrix)."""
    head, base = _read_header(path)
    size = os.path.getsize(path) - base

    def entry(key, dtype):
        if key not in head:
            raise KeyError(f"{key}: missing (is this weight NVFP4?)")
        e = head[key]
        if e["dtype"] not in dtype:
            raise ValueError(f"{key}: dtype {e['dtype']}, expected {dtype[0]}")
        lo, hi = e["data_offsets"]
        if hi > size:
            raise ValueError(f"{key}: data runs past the blob")
        return e, lo

    ce, c_lo = entry(name, ("U32", "I32"))
    if len(ce["shape"]) != 2:
        raise ValueError(f"{name}: expected a matrix, got {ce['shape']}")
    rows, words = ce["shape"]
    cols = words * 8
    if not 0 <= n0 <= n1 <= rows:
        raise ValueError(f"{name}: rows [{n0}, {n1}) outside a matrix of {rows}")
    se, s_lo = entry(name + ".scale", ("U8", "I8"))
    if list(se["shape"]) != [rows, cols // 16]:
        raise ValueError(f"{name}.scale: shape {se['shape']} does not fit {rows} x {cols}")
    ge, g_lo = entry(name + ".global_scale", ("F32",))
    if ge["data_offsets"][1] - g_lo < 4:
        raise ValueError("global scale is not four bytes")
    with open(path, "rb") as f:
        f.seek(base + c_lo + n0 * (cols // 2))
        wq = np.frombuffer(f.read((n1 - n0) * (cols // 2)), dtype=np.uint8).reshape(n1 - n0, cols // 2).copy()
        f.seek(base + s_lo + n0 * (cols // 16))
        ws = np.frombuffer(f.read((n1 - n0) * (cols // 16)), dtype=np.uint8).reshape(n1 - n0, cols // 16).copy()
        f.seek(base + g_lo)
        gs = np.frombuffer(f.read(4), dtype="<f4")[0]
    return wq, ws, np.full(n1 - n0, gs, dtype=np.float32), rows


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


# ---------------------------------------------------------------- the Ollama store around the blobs

def store_root() -> Path:
    """$OLLAMA_MODELS, else ~/.ollama/models (crates/lex-rt/src/qwen.rs:77-84)."""
    env = os.environ.get("OLLAMA_MODELS")
    return Path(env) if env else Path(os.environ.get("HOME", "")) / ".ollama" / "models"


def shard_span(rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [n0, n1) of rank `rank`: whole 128-row tiles, the remainder spread over the first ranks - the rule of
    lexb_shard_rows, restated so that a loader needs no device library."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if rows % 128:
        raise ValueError(f"sharding splits whole 128-row tiles; 128 does not divide {rows}")
    tiles = rows // 128
    base, extra = divmod(tiles, world)
    first = rank * base + min(rank, extra)
    return first * 128, (first + base + (1 if rank < extra else 0)) * 128


class Store:
    """A model in a local Ollama store: tensor names to blob paths (lex_rt::qwen::Store, crates/lex-rt/src/qwen.rs:70-145)."""

    def __init__(self, model: str, blobs: dict):
        self.model, self.blobs = model, blobs

    @classmethod
    def open(cls, model: str, root=None) -> "Store":
        """Open `name:tag` (default tag `latest`)."""
        name, _, tag = model.partition(":")
        root = Path(root) if root is not None else store_root()
        path = root / "manifests" / "registry.ollama.ai" / "library" / name / (tag or "latest")
        try:
            text = path.read_text()
        except OSError as e:
            raise FileNotFoundError(f"{model} is not in the Ollama store ({path}): {e}") from None
        layers = json.loads(text).get("layers")
        if not isinstance(layers, list):
            raise ValueError("manifest has no layers")
        blobs = {}
        for layer in layers:
            lname, digest = layer.get("name"), layer.get("digest")
            if not isinstance(lname, str) or not isinstance(digest, str):
                continue                                  # the licence and parameter layers carry no name
            blobs[lname] = root / "blobs" / digest.replace(":", "-")
        if not blobs:
            raise ValueError(f"{model} has no named tensors")
        return cls(model, blobs)

    def names(self) -> list[str]:
        return sorted(self.blobs)

    def has(self, name: str) -> bool:
        return name in self.blobs

    def _path(self, name: str) -> Path:
        if name not in self.blobs:
            raise KeyError(f"no tensor `{name}` in {self.model}")
        return self.blobs[name]

    def nvfp4(self, name: str, rows=None):
        """(wq, ws, wg) of a matrix, or of its rows [n0, n1) only."""
        path = self._path(name)
        if rows is None:
            return read_nvfp4(path, name)
        return read_nvfp4_rows(path, name, rows[0], rows[1])[:3]

    def rows_of(self, name: str) -> int:
        head, _ = _read_header(self._path(name))
        if name not in head:
            raise KeyError(f"{name}: not in its own blob")
        return int(head[name]["shape"][0])

    def nvfp4_shard(self, name: str, world: int, rank: int):
        """This rank's slab of a column-parallel matrix and its row span: (wq, ws, wg, n0, n1)."""
        n0, n1 = shard_span(self.rows_of(name), world, rank)
        return self.nvfp4(name, (n0, n1)) + (n0, n1)

    def gate_up_shard(self, gate: str, up: str, world: int, rank: int):
        """A rank's rows of gate and up, interleaved for the fused gate/up launch (row 2j = gate row j0 + j,
        row 2j + 1 = up row j0 + j): (wq, ws, wg, j0, j1) - the rank then owns activation columns [j0, j1).
        The span is dealt in whole 64-row tiles of each matrix, i.e. whole 128-row tiles of the interleaved one."""
        n = self.rows_of(gate)
        if self.rows_of(up) != n:
            raise ValueError("gate and up differ in rows")
        a0, a1 = shard_span(2 * n, world, rank)
        j0, j1 = a0 // 2, a1 // 2
        g, u = self.nvfp4(gate, (j0, j1)), self.nvfp4(up, (j0, j1))
        out = []
        for a, b in zip(g, u):
            both = np.empty((2 * (j1 - j0),) + a.shape[1:], dtype=a.dtype)
            both[0::2], both[1::2] = a, b
            out.append(both)
        return tuple(out) + (j0, j1)


def write_store(root, model: str, tensors: dict) -> None:
    """A synthetic store in the same layout (tests, synthetic checkpoints): one blob per matrix, named by the
    sha256 of its bytes, and a manifest whose layers name them."""
    root = Path(root)
    name, _, tag = model.partition(":")
    (root / "blobs").mkdir(parents=True, exist_ok=True)
    layers = [{"mediaType": "application/vnd.ollama.image.license", "digest": "sha256:0"}]   # a layer without a name
    for tname, triple in tensors.items():
        tmp = root / "blobs" / "tmp"
        write_nvfp4(tmp, {tname: triple})
        digest = hashlib.sha256(tmp.read_bytes()).hexdigest()
        tmp.rename(root / "blobs" / f"sha256-{digest}")
        layers.append({"mediaType": "application/vnd.ollama.image.tensor", "name": tname, "digest": f"sha256:{digest}"})
    mdir = root / "manifests" / "registry.ollama.ai" / "library" / name
    mdir.mkdir(parents=True, exist_ok=True)
    (mdir / (tag or "latest")).write_text(json.dumps({"schemaVersion": 2, "layers": layers}))
