"""B200 (sm_100a) backend for lex's `gemm_fp4` operator (and `matmul_q_x` with the NVFP4 layout, its small-batch sibling).

The compute lives in liblexb.so (CUDA, built from csrc/ by `python -m lex_gpu_b200.build`);
this package is its ctypes binding plus the synthetic-input generator and the n-sharded
multi-GPU wrapper.  Importing the package does not load the library; opening a Gpu does.
"""
from .device import Gpu, Buffer, Pipeline, HostBuffer, StepList, LexbError, load_library, shard_rows, prefill_chunks  # noqa: F401
from .gemm import Gemm, QBuf, GemmKernels, gemm_fp4, matmul_fp4, dequant_fp4_f16  # noqa: F401

__all__ = ["Gpu", "Buffer", "Pipeline", "HostBuffer", "StepList", "LexbError", "load_library", "shard_rows", "prefill_chunks",
           "Gemm", "QBuf", "GemmKernels", "gemm_fp4", "matmul_fp4", "dequant_fp4_f16"]
