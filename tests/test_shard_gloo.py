"""The n-sharded path with two ranks on CPU (gloo): each rank computes its row slab with the oracle,
the shards are all-gathered and assembled, and the result equals the unsharded product bit for bit.
This covers the host logic of the multi-GPU path (row ownership, gather layout, padding of unequal
shards); the kernels themselves are covered by the GPU tests."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, n: int, k: int, out_dir: str, op: str = "gemm_fp4"):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lex_gpu_b200 import inputs
    from lex_gpu_b200.shard import RowShard, all_gather_y, assemble
    from oracle import oracle as O
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=7)
    sh = RowShard.of(n, world, rank)
    q, s, g = sh.slice_weights(wq, ws, wg)
    fn = O.gemm_fp4 if op == "gemm_fp4" else O.matmul_q_x
    y_local = torch.from_numpy(fn(x, np.ascontiguousarray(q), np.ascontiguousarray(s), np.ascontiguousarray(g), threads=2))
    gathered = all_gather_y(y_local, sh)
    y = assemble(gathered, sh).numpy()
    if rank == 0:
        np.save(os.path.join(out_dir, "y.npy"), y)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n,world", [(512, 2), (384, 2)])        # equal shards; 2 tiles + 1 tile
def test_two_rank_sharded_product_equals_the_unsharded_one(tmp_path, n, world):
    m, k = 24, 256
    port = _free_port()
    mp.spawn(_worker, args=(world, port, m, n, k, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, str(ROOT))
    from lex_gpu_b200 import inputs
    from oracle import oracle as O
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=7)
    want = O.gemm_fp4(x, wq, ws, wg)
    got = np.load(tmp_path / "y.npy")
    assert np.array_equal(got, want)


def test_two_rank_sharded_decode_matmul(tmp_path):
    """The same row sharding for matmul_q_x (decode: 3 tokens), unequal shards."""
    m, n, k, world = 3, 384, 512, 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, m, n, k, str(tmp_path), "matmul_q_x"), nprocs=world, join=True)
    sys.path.insert(0, str(ROOT))
    from lex_gpu_b200 import inputs
    from oracle import oracle as O
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=7)
    assert np.array_equal(np.load(tmp_path / "y.npy"), O.matmul_q_x(x, wq, ws, wg))
