"""Loader for the reference's own CUDA kernels built by oracle/build_ref.py (oracle/_ref/*.so).

TEST INFRASTRUCTURE ONLY: the checker for the GPU tests and the "reference's kernel on this box" figure of the
benchmark.  The product package never imports this module.  The kernels are the reference's text compiled for
sm_100a: its emitted decode matvec (crates/lex-msl/tests/golden/matvec_nvfp4_17408x5120_cuda.cu) and
instances of its hand-scheduled GEMM (crates/lex-msl/src/gemm.rs:89-320).
"""
from __future__ import annotations

import ctypes
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"
_LIBS: dict[str, ctypes.CDLL] = {}


def gemm_entry(m: int, n: int, k: int, residual: bool = False) -> str:
    """The reference's name for the kernel (crates/lex-msl/src/gemm.rs:69-76), f16 activations."""
    return f"gemm_nvfp4_{m}x{n}x{k}{'_res' if residual else ''}_xh"


MATVEC_ENTRY = "matvec_nvfp4_17408x5120"


def available(entry: str) -> bool:
    return (REF / f"{entry}.so").exists()


def built_entries() -> list[str]:
    return sorted(p.stem for p in REF.glob("*.so"))


def _lib(entry: str) -> ctypes.CDLL:
    if entry not in _LIBS:
        path = REF / f"{entry}.so"
        if not path.exists():
            raise FileNotFoundError(f"{path} is missing: run `python oracle/build_ref.py` where the reference tree is present")
        lib = ctypes.CDLL(str(path))
        lib.lexref_launch.restype = ctypes.c_int
        lib.lexref_launch.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p]
        lib.lexref_info.restype = ctypes.c_char_p
        _LIBS[entry] = lib
    return _LIBS[entry]


def info(entry: str) -> str:
    return _lib(entry).lexref_info().decode()


def launch(entry: str, device_ptrs: list[int], stream: int = 0) -> None:
    """One launch with positional device pointers [x, wq, ws, wg, (r), y] on a CUDA stream handle."""
    arr = (ctypes.c_void_p * len(device_ptrs))(*device_ptrs)
    rc = _lib(entry).lexref_launch(arr, len(device_ptrs), ctypes.c_void_p(stream))
    if rc != 0:
        raise RuntimeError(f"{entry}: launch failed with CUDA error {rc}")


def run_torch(entry: str, tensors: list, stream=None) -> None:
    """Launch on torch tensors (all on one CUDA device, contiguous), on torch's current stream by default."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
    launch(entry, [t.data_ptr() for t in tensors], s)


def gemm(x16, wq, ws, wg, r=None):
    """y f32[m, n] of the reference's GEMM kernel for numpy inputs (x as float16)."""
    import numpy as np
    import torch
    m, k = x16.shape
    n = wq.shape[0]
    entry = gemm_entry(m, n, k, r is not None)
    dev = torch.device("cuda", torch.cuda.current_device())
    tx = torch.from_numpy(np.ascontiguousarray(x16).view(np.int16)).to(dev)
    tq, ts = (torch.from_numpy(np.ascontiguousarray(a).view(np.uint8)).to(dev) for a in (wq, ws))
    tg = torch.from_numpy(np.ascontiguousarray(wg, dtype=np.float32)).to(dev)
    ty = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
    bufs = [tx, tq, ts, tg]
    if r is not None:
        bufs.append(torch.from_numpy(np.ascontiguousarray(r, dtype=np.float32)).to(dev))
    run_torch(entry, bufs + [ty])
    torch.cuda.synchronize(dev)
    return ty.cpu().numpy()


def matvec(x32, wq, ws, wg):
    """y f32[1, 17408] of the reference's emitted decode matvec (x f32[1, 5120])."""
    import numpy as np
    import torch
    assert x32.shape == (1, 5120) and wq.shape == (17408, 2560)
    dev = torch.device("cuda", torch.cuda.current_device())
    tx = torch.from_numpy(np.ascontiguousarray(x32, dtype=np.float32)).to(dev)
    tq, ts = (torch.from_numpy(np.ascontiguousarray(a).view(np.uint8)).to(dev) for a in (wq, ws))
    tg = torch.from_numpy(np.ascontiguousarray(wg, dtype=np.float32)).to(dev)
    ty = torch.full((1, 17408), float("nan"), dtype=torch.float32, device=dev)
    run_torch(MATVEC_ENTRY, [tx, tq, ts, tg, ty])
    torch.cuda.synchronize(dev)
    return ty.cpu().numpy()
