"""ctypes binding of liblexb's C ABI, shaped like lex_cuda::device
(crates/lex-cuda/src/device.rs): Gpu, Buffer, Pipeline, Step, run_launches, run_each_timed.

This module is only a binding.  Every operation goes through the shared library built from
csrc/; there is no Python or CPU implementation behind it, and loading fails with an error
when the library is missing.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char, c_double, c_int, c_size_t, c_uint8, c_uint32, c_uint64, c_void_p
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "liblexb.so"

KERNEL_AUTO, KERNEL_MATVEC, KERNEL_TCGEN05, KERNEL_TCGEN05_PAIR = 0, 1, 2, 3
STATUS_WAIT_NEVER = 1 << 16

# Every symbol include/lexb.h declares.
SYMBOLS = [
    "lexb_last_error", "lexb_version", "lexb_open", "lexb_close", "lexb_info", "lexb_set_stream", "lexb_get_stream",
    "lexb_sync", "lexb_alloc", "lexb_zeroed", "lexb_wrap", "lexb_free", "lexb_buffer_ptr", "lexb_buffer_bytes",
    "lexb_upload", "lexb_download", "lexb_memset", "lexb_host_alloc", "lexb_host_free", "lexb_gemm_fp4_plan",
    "lexb_pipeline_free", "lexb_pipeline_describe", "lexb_gemm_fp4_launch", "lexb_gemm_fp4_run_host",
    "lexb_gemm_fp4_enqueue_host",
    "lexb_run_launches", "lexb_list_runs", "lexb_run_each_timed", "lexb_time_launches", "lexb_status_word",
    "lexb_selftest_bounded_wait", "lexb_dequant_fp4_f16", "lexb_shard_rows", "lexb_trace_enable", "lexb_trace_read",
    "lexb_gemm_fp4_splitk_static", "lexb_gemm_fp4_launch_gather", "lexb_silu_mul", "lexb_prefill_chunks",
    "lexb_matmul_fp4_plan", "lexb_debug_fail_next", "lexb_gemm_fp4_silu_launch", "lexb_gemm_fp4_silu_launch_gather",
    "lexb_interleave_rows", "lexb_quant16", "lexb_matmul_int8_plan",
]


class LexbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"lexb error {code}: {message}")
        self.code = code
        self.message = message


class DeviceInfo(ctypes.Structure):
    _fields_ = [("name", c_char * 128), ("cc_major", c_int), ("cc_minor", c_int), ("sm_count", c_int),
                ("unified_memory", c_int), ("max_threadgroup_bytes", c_size_t),
                ("recommended_working_set_bytes", c_uint64), ("l2_bytes", c_size_t)]


class Sched(ctypes.Structure):
    _fields_ = [("kernel", c_uint32), ("tm", c_uint32), ("stages", c_uint32), ("kc", c_uint32), ("w_stages", c_uint32), ("k_splits", c_uint32),
                ("flags", c_uint32)]


SCHED_WEIGHTS_MAY_CHANGE = 1
SCHED_WEIGHTS_CONSTANT = 2
SITE_ALLOC, SITE_COPY, SITE_LAUNCH, SITE_ENCODE = 1, 2, 3, 4


class Lowered(ctypes.Structure):
    _fields_ = [("entry", c_char * 96), ("grid", c_uint32), ("grid2", c_uint32), ("threads", c_uint32),
                ("threadgroup_bytes", c_uint32), ("nbind", c_uint32), ("writes", c_uint8 * 8), ("kernel", c_uint32),
                ("m", c_uint32), ("n", c_uint32), ("k", c_uint32), ("residual", c_uint32),
                ("bm", c_uint32), ("bn", c_uint32), ("bk", c_uint32), ("stages", c_uint32),
                ("k_splits", c_uint32), ("scratch_bytes", c_uint64)]


class StepStruct(ctypes.Structure):
    _fields_ = [("pipeline", c_void_p), ("buffers", POINTER(c_void_p)), ("nbuffers", c_uint32)]


_lib = None


def load_library() -> ctypes.CDLL:
    """Load liblexb.so from the package directory.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m lex_gpu_b200.build` "
                           "(there is no CPU or Python implementation to fall back to)")
    L = ctypes.CDLL(str(LIB_PATH))
    vp, u32, sz = c_void_p, c_uint32, c_size_t
    L.lexb_last_error.restype = ctypes.c_char_p
    L.lexb_version.restype = ctypes.c_char_p
    L.lexb_open.argtypes = [c_int, POINTER(vp)]
    L.lexb_close.argtypes = [vp]
    L.lexb_close.restype = None
    L.lexb_info.argtypes = [vp, POINTER(DeviceInfo)]
    L.lexb_set_stream.argtypes = [vp, vp]
    L.lexb_get_stream.argtypes = [vp]
    L.lexb_get_stream.restype = vp
    L.lexb_sync.argtypes = [vp]
    L.lexb_alloc.argtypes = [vp, sz, POINTER(vp)]
    L.lexb_zeroed.argtypes = [vp, sz, POINTER(vp)]
    L.lexb_wrap.argtypes = [vp, vp, sz, POINTER(vp)]
    L.lexb_free.argtypes = [vp]
    L.lexb_buffer_ptr.argtypes = [vp]
    L.lexb_buffer_ptr.restype = vp
    L.lexb_buffer_bytes.argtypes = [vp]
    L.lexb_buffer_bytes.restype = sz
    L.lexb_upload.argtypes = [vp, vp, sz, vp, sz]
    L.lexb_download.argtypes = [vp, vp, sz, vp, sz]
    L.lexb_memset.argtypes = [vp, vp, c_int, sz]
    L.lexb_host_alloc.argtypes = [sz, POINTER(vp)]
    L.lexb_host_free.argtypes = [vp]
    L.lexb_gemm_fp4_plan.argtypes = [vp, u32, u32, u32, c_int, POINTER(Sched), POINTER(vp)]
    L.lexb_matmul_fp4_plan.argtypes = [vp, u32, u32, u32, c_int, c_int, POINTER(Sched), POINTER(vp)]
    L.lexb_pipeline_free.argtypes = [vp]
    L.lexb_pipeline_free.restype = None
    L.lexb_pipeline_describe.argtypes = [vp, POINTER(Lowered)]
    L.lexb_gemm_fp4_launch.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp]
    L.lexb_gemm_fp4_run_host.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    L.lexb_gemm_fp4_enqueue_host.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    L.lexb_run_launches.argtypes = [vp, POINTER(StepStruct), sz, POINTER(c_double), POINTER(c_double)]
    L.lexb_run_each_timed.argtypes = [vp, POINTER(StepStruct), sz, POINTER(c_double)]
    L.lexb_time_launches.argtypes = [vp, POINTER(StepStruct), sz, u32, POINTER(c_double)]
    L.lexb_list_runs.argtypes = [vp, POINTER(StepStruct), sz, POINTER(c_uint32)]
    L.lexb_status_word.argtypes = [vp, POINTER(u32)]
    L.lexb_selftest_bounded_wait.argtypes = [vp, u32]
    L.lexb_dequant_fp4_f16.argtypes = [vp, u32, u32, vp, vp, vp, vp]
    L.lexb_shard_rows.argtypes = [u32, u32, u32, POINTER(u32), POINTER(u32)]
    L.lexb_trace_enable.argtypes = [vp, u32]
    L.lexb_silu_mul.argtypes = [vp, u32, u32, vp, sz, sz, vp, sz, sz, vp, c_int]
    L.lexb_prefill_chunks.argtypes = [u32, u32, c_int, POINTER(u32), u32, POINTER(u32)]
    L.lexb_gemm_fp4_launch_gather.argtypes = [vp, vp, vp, vp, vp, vp, vp, POINTER(vp), u32, u32, u32]
    L.lexb_gemm_fp4_splitk_static.argtypes = [vp, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp]
    L.lexb_trace_read.argtypes = [vp, vp, u32]
    L.lexb_debug_fail_next.argtypes = [c_int, c_int, c_int]
    L.lexb_gemm_fp4_silu_launch.argtypes = [vp, vp, vp, vp, vp, vp, vp]
    L.lexb_gemm_fp4_silu_launch_gather.argtypes = [vp, vp, vp, vp, vp, vp, POINTER(vp), u32, u32, u32]
    L.lexb_interleave_rows.argtypes = [vp, vp, vp, sz, sz, vp]
    L.lexb_quant16.argtypes = [vp, u32, u32, c_int, vp, vp, vp]
    L.lexb_matmul_int8_plan.argtypes = [vp, u32, u32, u32, c_int, POINTER(Sched), POINTER(vp)]
    _lib = L
    return L


def _check(rc: int) -> None:
    if rc != 0:
        raise LexbError(rc, load_library().lexb_last_error().decode(errors="replace"))


def debug_fail_next(site: int, nth: int = 1, cuda_error: int = 0) -> None:
    """Tests of the error paths: the nth call from now that reaches `site` (SITE_ALLOC, SITE_COPY, SITE_LAUNCH,
    SITE_ENCODE) reports a CUDA error instead of being made; site 0 disarms everything."""
    _check(load_library().lexb_debug_fail_next(site, nth, cuda_error))


def prefill_chunks(tokens: int, limit: int = 0, gemm_ok: bool = True) -> list[int]:
    """How lex-rt cuts a prompt into prefill chunks (host arithmetic only; needs no GPU)."""
    L = load_library()
    count = c_uint32()
    _check(L.lexb_prefill_chunks(tokens, limit, int(gemm_ok), None, 0, byref(count)))
    arr = (c_uint32 * max(count.value, 1))()
    _check(L.lexb_prefill_chunks(tokens, limit, int(gemm_ok), arr, count.value, byref(count)))
    return [arr[i] for i in range(count.value)]


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [n0, n1) of W that `rank` of `world` owns (host arithmetic only; needs no GPU)."""
    n0, n1 = c_uint32(), c_uint32()
    _check(load_library().lexb_shard_rows(n, world, rank, byref(n0), byref(n1)))
    return n0.value, n1.value


class Buffer:
    """A device buffer (lex_cuda::Buffer, device.rs:257-278); freed on close() or collection."""

    def __init__(self, gpu: "Gpu", handle: int, keepalive=None):
        self.gpu, self._h, self._keep = gpu, handle, keepalive

    @property
    def handle(self) -> int:
        if self._h is None:
            raise LexbError(1, "buffer already freed")
        return self._h

    def len_bytes(self) -> int:
        return int(load_library().lexb_buffer_bytes(self.handle))

    @property
    def ptr(self) -> int:
        return int(load_library().lexb_buffer_ptr(self.handle) or 0)

    def close(self) -> None:
        if self._h is not None:
            load_library().lexb_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Pipeline:
    """A planned kernel and its launch shape (lex_cuda::Pipeline, device.rs:281-301)."""

    def __init__(self, gpu: "Gpu", handle: int):
        self.gpu, self._h = gpu, handle

    @property
    def handle(self) -> int:
        if self._h is None:
            raise LexbError(1, "pipeline already freed")
        return self._h

    def describe(self) -> Lowered:
        out = Lowered()
        _check(load_library().lexb_pipeline_describe(self.handle, byref(out)))
        return out

    def close(self) -> None:
        if self._h is not None:
            load_library().lexb_pipeline_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


Step = tuple  # (Pipeline, [Buffer, ...]) in the order [x, wq, ws, wg, (r), y]; device.rs:314


class StepList:
    """A step list marshalled once (the C array of lexb_step): pass it to run_launches / run_each_timed /
    time_launches instead of the Python list when the same list is issued repeatedly or is being timed."""

    def __init__(self, steps: Sequence[Step]):
        self.n = len(steps)
        self.arr = (StepStruct * max(self.n, 1))()
        self._keep = []
        for i, (pipe, bufs) in enumerate(steps):
            ptrs = (c_void_p * len(bufs))(*[b.handle for b in bufs])
            self._keep.append(ptrs)
            self.arr[i].pipeline = pipe.handle
            self.arr[i].buffers = ctypes.cast(ptrs, POINTER(c_void_p))
            self.arr[i].nbuffers = len(bufs)


class Gpu:
    """lex_cuda::Gpu (device.rs:316-810) for the one operator this backend provides."""

    def __init__(self, device: int = 0):
        self._L = load_library()
        h = c_void_p()
        _check(self._L.lexb_open(device, byref(h)))
        self._h = h.value
        self.device = device

    @classmethod
    def open(cls, device: int = 0) -> "Gpu":
        return cls(device)

    @property
    def handle(self) -> int:
        if self._h is None:
            raise LexbError(1, "gpu already closed")
        return self._h

    def close(self) -> None:
        if self._h is not None:
            self._L.lexb_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def info(self) -> DeviceInfo:
        out = DeviceInfo()
        _check(self._L.lexb_info(self.handle, byref(out)))
        return out

    def name(self) -> str:
        return self.info().name.decode()

    def set_stream(self, cuda_stream: Optional[int]) -> None:
        """None: the library's own stream.  An integer is a CUDA stream handle as torch gives it
        (`torch.cuda.current_stream().cuda_stream`); 0, torch's default stream, is passed on as
        cudaStreamLegacy (0x1), because a null handle means the own stream to the library."""
        if cuda_stream is None:
            h = 0
        else:
            h = cuda_stream or 1
        _check(self._L.lexb_set_stream(self.handle, c_void_p(h)))

    def sync(self) -> None:
        _check(self._L.lexb_sync(self.handle))

    # ---- memory
    def alloc(self, nbytes: int) -> Buffer:
        h = c_void_p()
        _check(self._L.lexb_alloc(self.handle, nbytes, byref(h)))
        return Buffer(self, h.value)

    def zeroed(self, nbytes: int) -> Buffer:
        h = c_void_p()
        _check(self._L.lexb_zeroed(self.handle, nbytes, byref(h)))
        return Buffer(self, h.value)

    def upload(self, array: np.ndarray) -> Buffer:
        a = np.ascontiguousarray(array)
        b = self.alloc(a.nbytes)
        self.write(b, 0, a)
        return b

    def wrap(self, device_ptr: int, nbytes: int, keepalive=None) -> Buffer:
        """A non-owning view of device memory allocated elsewhere (e.g. a torch tensor)."""
        h = c_void_p()
        _check(self._L.lexb_wrap(self.handle, c_void_p(device_ptr), nbytes, byref(h)))
        return Buffer(self, h.value, keepalive)

    def wrap_tensor(self, t) -> Buffer:
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("wrap_tensor needs a contiguous CUDA tensor")
        return self.wrap(t.data_ptr(), t.numel() * t.element_size(), keepalive=t)

    def write(self, buf: Buffer, byte_offset: int, array: np.ndarray) -> None:
        a = np.ascontiguousarray(array)
        _check(self._L.lexb_upload(self.handle, buf.handle, byte_offset, c_void_p(a.ctypes.data), a.nbytes))

    def download(self, buf: Buffer, dtype, shape, byte_offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        _check(self._L.lexb_download(self.handle, buf.handle, byte_offset, c_void_p(out.ctypes.data), out.nbytes))
        return out

    def memset(self, buf: Buffer, byte: int, nbytes: Optional[int] = None) -> None:
        _check(self._L.lexb_memset(self.handle, buf.handle, byte, buf.len_bytes() if nbytes is None else nbytes))

    # ---- the operator
    def plan_gemm_fp4(self, m: int, n: int, k: int, residual: bool = False, kernel: int = 0, tm: int = 0,
                      stages: int = 0, kc: int = 0, w_stages: int = 0, k_splits: int = 0, weights_constant: bool = False,
                      weights_may_change: bool = False) -> Pipeline:
        flags = (SCHED_WEIGHTS_MAY_CHANGE if weights_may_change else 0) | (SCHED_WEIGHTS_CONSTANT if weights_constant else 0)
        s = Sched(kernel, tm, stages, kc, w_stages, k_splits, flags)
        h = c_void_p()
        _check(self._L.lexb_gemm_fp4_plan(self.handle, m, n, k, int(residual), byref(s), byref(h)))
        return Pipeline(self, h.value)

    def plan_matmul_fp4(self, t: int, n_out: int, n_in: int, residual: bool = False, x_half: bool = True,
                        stages: int = 0, k_splits: int = 0, weights_may_change: bool = False,
                        weights_constant: bool = False) -> Pipeline:
        """matmul_q_x with the NVFP4 layout for t <= 32 tokens (llama.rs:444-499): weights as f32, not
        rounded to f16; runs on the block-scaled FP4 tensor-core path.  Launches are in order on their stream;
        `weights_constant` promises that nothing writes wq/ws while launches are in flight, so that a launch
        made on its own may load them ahead of the stream's order (inside a step list the library works that
        out itself unless `weights_may_change`)."""
        flags = (SCHED_WEIGHTS_MAY_CHANGE if weights_may_change else 0) | (SCHED_WEIGHTS_CONSTANT if weights_constant else 0)
        s = Sched(0, 0, stages, 0, 0, k_splits, flags)
        h = c_void_p()
        _check(self._L.lexb_matmul_fp4_plan(self.handle, t, n_out, n_in, int(residual), int(x_half), byref(s), byref(h)))
        return Pipeline(self, h.value)

    def plan_matmul_int8(self, t: int, n_out: int, n_in: int, residual: bool = False, stages: int = 0, k_splits: int = 0) -> Pipeline:
        """matmul_int8 (crates/lex-msl/src/int8.rs:121-223): int16 activations with one f32 scale per 16, as quant16
        leaves them; launched as a step with the bindings [xq, xs, wq, ws, wg, (r), y]."""
        s = Sched(0, 0, stages, 0, 0, k_splits, 0)
        h = c_void_p()
        _check(self._L.lexb_matmul_int8_plan(self.handle, t, n_out, n_in, int(residual), byref(s), byref(h)))
        return Pipeline(self, h.value)

    def quant16(self, m: int, k: int, x: Buffer, xq: Buffer, xs: Buffer, x_half: bool) -> None:
        """quant16 (crates/lex-msl/src/int8.rs:47-114): x[m, k] -> int16 xq[m, k] and f32 xs[m, k/16]."""
        _check(self._L.lexb_quant16(self.handle, m, k, int(x_half), x.handle, xq.handle, xs.handle))

    def run(self, pipe: Pipeline, bufs: Sequence[Buffer]) -> None:
        """One launch, asynchronous; bufs = [x, wq, ws, wg, (r), y] (Gpu::run, device.rs:629-648)."""
        res = len(bufs) == 6
        if len(bufs) not in (5, 6):
            raise LexbError(1, f"gemm_fp4 binds 5 or 6 buffers, not {len(bufs)}")
        x, wq, ws, wg = bufs[:4]
        r, y = (bufs[4], bufs[5]) if res else (None, bufs[4])
        _check(self._L.lexb_gemm_fp4_launch(self.handle, pipe.handle, x.handle, wq.handle, ws.handle, wg.handle,
                                            r.handle if r is not None else None, y.handle))

    def run_gather(self, pipe: Pipeline, x: Buffer, wq: Buffer, ws: Buffer, wg: Buffer, r: Optional[Buffer],
                   y_ptr_of_rank: Sequence[int], n_total: int, n0: int) -> None:
        """One launch whose epilogue stores this rank's columns [n0, n0+n) into every rank's gathered y
        (device addresses valid on this GPU, e.g. symmetric-memory peer pointers).  Asynchronous."""
        arr = (c_void_p * len(y_ptr_of_rank))(*[c_void_p(p) for p in y_ptr_of_rank])
        _check(self._L.lexb_gemm_fp4_launch_gather(self.handle, pipe.handle, x.handle, wq.handle, ws.handle, wg.handle,
                                                   r.handle if r is not None else None, arr, len(y_ptr_of_rank),
                                                   n_total, n0))

    def run_silu(self, pipe: Pipeline, x: Buffer, wq: Buffer, ws: Buffer, wg: Buffer, act: Buffer) -> None:
        """gate/up in one launch with silu(gate) * up fused in: wq/ws/wg hold gate and up rows interleaved, act is
        f16 [m, n/2] (lexb_gemm_fp4_silu_launch)."""
        _check(self._L.lexb_gemm_fp4_silu_launch(self.handle, pipe.handle, x.handle, wq.handle, ws.handle, wg.handle, act.handle))

    def run_silu_gather(self, pipe: Pipeline, x: Buffer, wq: Buffer, ws: Buffer, wg: Buffer, act_ptrs: Sequence[int],
                        n_total: int, n0: int) -> None:
        """The n-sharded form with the all-gather of the f16 activation fused in (peer stores)."""
        arr = (c_void_p * len(act_ptrs))(*act_ptrs)
        _check(self._L.lexb_gemm_fp4_silu_launch_gather(self.handle, pipe.handle, x.handle, wq.handle, ws.handle, wg.handle,
                                                        arr, len(act_ptrs), n_total, n0))

    def interleave_rows(self, a: Buffer, b: Buffer, rows: int, row_bytes: int, out: Buffer) -> None:
        """out row 2j = a row j, out row 2j + 1 = b row j, on the device (lexb_interleave_rows)."""
        _check(self._L.lexb_interleave_rows(self.handle, a.handle, b.handle, rows, row_bytes, out.handle))

    def enqueue_host(self, pipe: Pipeline, x_host_ptr: int, x_dev: Buffer, wq: Buffer, ws: Buffer, wg: Buffer,
                     r: Optional[Buffer], y_dev: Buffer, y_host_ptr: int) -> None:
        """run_host without the wait: copy in, launch, copy out on the current stream; sync() before using y."""
        _check(self._L.lexb_gemm_fp4_enqueue_host(self.handle, pipe.handle, c_void_p(x_host_ptr), x_dev.handle, wq.handle,
                                                  ws.handle, wg.handle, r.handle if r is not None else None,
                                                  y_dev.handle, c_void_p(y_host_ptr)))

    def run_host(self, pipe: Pipeline, x_host_ptr: int, x_dev: Buffer, wq: Buffer, ws: Buffer, wg: Buffer,
                 r: Optional[Buffer], y_dev: Buffer, y_host_ptr: int) -> None:
        _check(self._L.lexb_gemm_fp4_run_host(self.handle, pipe.handle, c_void_p(x_host_ptr), x_dev.handle, wq.handle,
                                              ws.handle, wg.handle, r.handle if r is not None else None,
                                              y_dev.handle, c_void_p(y_host_ptr)))

    def run_launches(self, steps: Sequence[Step]) -> tuple[float, float]:
        s = steps if isinstance(steps, StepList) else StepList(steps)
        cpu, wall = c_double(), c_double()
        _check(self._L.lexb_run_launches(self.handle, s.arr, s.n, byref(cpu), byref(wall)))
        return cpu.value, wall.value

    def run_each_timed(self, steps: Sequence[Step]) -> list[float]:
        s = steps if isinstance(steps, StepList) else StepList(steps)
        out = (c_double * max(s.n, 1))()
        _check(self._L.lexb_run_each_timed(self.handle, s.arr, s.n, out))
        return [out[i] for i in range(s.n)]

    def time_launches(self, steps: Sequence[Step], reps: int = 1) -> float:
        s = steps if isinstance(steps, StepList) else StepList(steps)
        out = c_double()
        _check(self._L.lexb_time_launches(self.handle, s.arr, s.n, reps, byref(out)))
        return out.value

    def list_runs(self, steps: Sequence[Step]) -> list:
        """For every step the number of steps of the launch `run_launches` would put it in (1: its own)."""
        s = steps if isinstance(steps, StepList) else StepList(steps)
        out = (c_uint32 * max(s.n, 1))()
        _check(self._L.lexb_list_runs(self.handle, s.arr, s.n, out))
        return list(out[:s.n])

    def status_word(self) -> int:
        out = c_uint32()
        _check(self._L.lexb_status_word(self.handle, byref(out)))
        return out.value

    def gemm_fp4_splitk_static(self, m: int, n: int, k: int, k_splits: int, bufs: Sequence[Buffer]) -> None:
        """Split-K GEMM whose workspace is the library's built-in array: allocates nothing.
        bufs = [x, wq, ws, wg, (r), y]; asynchronous on the gpu's stream."""
        if len(bufs) not in (5, 6):
            raise LexbError(1, f"gemm_fp4 binds 5 or 6 buffers, not {len(bufs)}")
        x, wq, ws, wg = bufs[:4]
        r, y = (bufs[4], bufs[5]) if len(bufs) == 6 else (None, bufs[4])
        _check(self._L.lexb_gemm_fp4_splitk_static(self.handle, m, n, k, k_splits, x.handle, wq.handle, ws.handle,
                                                   wg.handle, r.handle if r is not None else None, y.handle))

    def silu_mul(self, rows: int, cols: int, gate: Buffer, up: Buffer, out: Buffer, out_f16: bool = True,
                 gate_offset: int = 0, gate_pitch: int = 0, up_offset: int = 0, up_pitch: int = 0) -> None:
        """out = silu(gate) * up; offsets and pitches in f32 elements (pitch 0 = cols)."""
        _check(self._L.lexb_silu_mul(self.handle, rows, cols, gate.handle, gate_offset, gate_pitch or cols, up.handle,
                                     up_offset, up_pitch or cols, out.handle, int(out_f16)))

    def trace_enable(self, max_ctas: int) -> None:
        _check(self._L.lexb_trace_enable(self.handle, max_ctas))

    def trace_read(self, ctas: int) -> np.ndarray:
        """uint64 [ctas, 16] phase timers of the last traced launch (see lexb_trace_enable)."""
        out = np.zeros((ctas, 16), dtype=np.uint64)
        _check(self._L.lexb_trace_read(self.handle, c_void_p(out.ctypes.data), ctas))
        return out

    def selftest_bounded_wait(self, limit_us: int = 1000) -> None:
        _check(self._L.lexb_selftest_bounded_wait(self.handle, limit_us))

    def dequant_fp4_f16(self, n: int, k: int, wq: Buffer, ws: Buffer, wg: Buffer, out: Buffer) -> None:
        _check(self._L.lexb_dequant_fp4_f16(self.handle, n, k, wq.handle, ws.handle, wg.handle, out.handle))


class HostBuffer:
    """Page-locked host memory viewed as a numpy array."""

    def __init__(self, nbytes: int):
        p = c_void_p()
        _check(load_library().lexb_host_alloc(nbytes, byref(p)))
        self.ptr, self.nbytes = p.value, nbytes

    def array(self, dtype, shape) -> np.ndarray:
        buf = (ctypes.c_uint8 * self.nbytes).from_address(self.ptr)
        return np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def close(self) -> None:
        if self.ptr:
            load_library().lexb_host_free(c_void_p(self.ptr))
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
