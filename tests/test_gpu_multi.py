"""Two or more GPUs: the fused all-gather epilogue over symmetric memory against the NCCL all-gather.
Skipped on a single-GPU machine (the store logic itself is covered there with several buffers on one GPU)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import lex_gpu_b200 as L
    from lex_gpu_b200 import inputs
    from lex_gpu_b200.shard import RowShard, SymmetricY, all_gather_y, assemble
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=9)
    sh = RowShard.of(n, world, rank)
    q_, s_, g_ = sh.slice_weights(wq, ws, wg)
    gpu = L.Gpu(rank)
    stream = torch.cuda.current_stream()
    gpu.set_stream(stream.cuda_stream)
    q = L.QBuf(gpu, np.ascontiguousarray(q_), np.ascontiguousarray(s_), np.ascontiguousarray(g_))
    xb = gpu.upload(x)
    pipe = gpu.plan_gemm_fp4(m, sh.rows, k, kernel=3)
    # NCCL path
    y_local = torch.empty((m, sh.rows), dtype=torch.float32, device="cuda")
    gpu.run(pipe, q.bind(xb, None, gpu.wrap_tensor(y_local)))
    y_nccl = assemble(all_gather_y(y_local, sh), sh)
    # fused path
    sy = SymmetricY(m, n, dist.group.WORLD)
    sy.tensor.fill_(float("nan"))
    sy.barrier()
    gpu.run_gather(pipe, xb, q.wq, q.ws, q.wg, None, sy.ptrs, n, sh.n0)
    sy.barrier()
    torch.cuda.synchronize()
    same = torch.equal(sy.tensor, y_nccl)
    if rank == 0:
        np.save(os.path.join(out_dir, "y.npy"), sy.tensor.cpu().numpy())
    flag = torch.tensor([1 if same else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        np.save(os.path.join(out_dir, "same.npy"), flag.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("shape", ["whole tiles", "27B gate/up shard"])
def test_fused_gather_equals_nccl_all_gather(tmp_path, shape):
    """Every rank's gathered y, written by the other ranks' peer stores, equals the NCCL all-gather of the same
    shards bit for bit and the oracle to tolerance.  The second shape is what each rank of an n-sharded 27B
    gate/up call computes (2176 rows, k = 5120: the planner splits K, so the stores come from the reduction
    launch)."""
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)        # every GPU of the box: the gather takes up to 8 ranks
    if world < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = (512, 256 * world * 2, 1024) if shape == "whole tiles" else (512, 2176 * world, 5120)
    mp.spawn(_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, str(ROOT))
    from lex_gpu_b200 import inputs
    from oracle import oracle as O
    assert int(np.load(tmp_path / "same.npy")[0]) == 1
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=9)
    err, scale, rel = O.err_of_scale(np.load(tmp_path / "y.npy"), O.gemm_fp4(x, wq, ws, wg))
    assert scale > 1e-3 and err <= 2e-3 and rel <= (2e-3 if k < 4096 else 1e-2)


def _decode_worker(rank, world, port, m, n, k, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import lex_gpu_b200 as L
    from lex_gpu_b200 import inputs
    from lex_gpu_b200.shard import RowShard, all_gather_y, assemble
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=11)
    sh = RowShard.of(n, world, rank)
    q_, s_, g_ = sh.slice_weights(wq, ws, wg)
    gpu = L.Gpu(rank)
    gpu.set_stream(torch.cuda.current_stream().cuda_stream)
    q = L.QBuf(gpu, np.ascontiguousarray(q_), np.ascontiguousarray(s_), np.ascontiguousarray(g_))
    xb = gpu.upload(x)
    pipe = gpu.plan_matmul_fp4(m, sh.rows, k)
    y_local = torch.empty((m, sh.rows), dtype=torch.float32, device="cuda")
    steps = [(pipe, q.bind(xb, None, gpu.wrap_tensor(y_local)))] * 3        # a short step list: the hint path too
    gpu.run_launches(steps)
    y = assemble(all_gather_y(y_local, sh), sh)
    if rank == 0:
        np.save(os.path.join(out_dir, "y_decode.npy"), y.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_row_sharded_decode_matmul(tmp_path):
    """matmul_q_x with the rows of W split over the GPUs and the shards gathered by NCCL."""
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)        # every GPU of the box: the gather takes up to 8 ranks
    if world < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = 3, 128 * world * 3, 2048
    mp.spawn(_decode_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, str(ROOT))
    from lex_gpu_b200 import inputs
    from oracle import oracle as O
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=11)
    err, scale, _ = O.err_of_scale(np.load(tmp_path / "y_decode.npy"), O.matmul_q_x(x, wq, ws, wg))
    assert scale > 1e-3 and err <= 1e-4
