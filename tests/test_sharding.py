"""The M-sharding of the path, on CPU: the shard arithmetic, and a world-size-2 gloo run in which each rank
computes its own row block with the oracle and the blocks are all-gathered in rank order."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from gpurs_b200.sharding import equal_shards, row_shard, shard_table

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("m", [0, 1, 127, 128, 129, 1000, 8192, 16384, 8192 * 8 + 5])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_shards_partition_the_rows(m, world):
    table = shard_table(m, world)
    position = 0
    for first, rows in table:
        assert first == position and rows >= 0
        position += rows
    assert position == m
    # every boundary except the end is on a tile boundary
    assert all(first % 128 == 0 for first, rows in table if rows)
    counts = [rows for _, rows in table]
    assert max(counts) - min(counts) <= 128 + 127


def test_configurations_shard_evenly():
    for world in (1, 2, 4, 8):
        assert equal_shards(8192, world)            # int8 8192^3 across 1/2/4/8
        assert row_shard(8192, world, world - 1) == (8192 - 8192 // world, 8192 // world)
    assert shard_table(16384, 8) == [(2048 * r, 2048) for r in range(8)]   # the sparse configuration
    assert not equal_shards(1000, 3)
    with pytest.raises(ValueError):
        row_shard(10, 2, 2)


WORKER = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch, torch.distributed as dist
import oracle as O
from gpurs_b200.sharding import row_shard
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
rank, world = dist.get_rank(), dist.get_world_size()
m, n, k = 512, 96, 160
a, b = O.fill_int8(m * k, 1), O.fill_int8(n * k, 2)           # the same seeded operands on every rank
first, rows = row_shard(m, world, rank)
mine = O.matmul_rows_i8(a, b, n, k, np.arange(first, first + rows))   # only this rank's rows of A are read
block = torch.from_numpy(mine.astype(np.int32))
gathered = torch.empty((m, n), dtype=torch.int32)
dist.all_gather_into_tensor(gathered, block)                  # blocks land in rank order
full = O.matmul_rows_i8(a, b, n, k, np.arange(m)).astype(np.int32)
ok = bool((gathered.numpy() == full).all())
flag = torch.tensor([1 if ok else 0]); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.barrier(); dist.destroy_process_group()
sys.exit(0 if flag.item() == 1 else 1)
"""


def test_two_rank_gloo_shard_and_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = str(29600 + os.getpid() % 300)
    workers = [subprocess.Popen([sys.executable, str(script), str(ROOT), port, str(rank)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
               for rank in range(2)]
    for worker in workers:
        output, _ = worker.communicate(timeout=240)
        assert worker.returncode == 0, output.decode()[-2000:]


COMM_WORKER = r"""
import sys
sys.path.insert(0, sys.argv[1])
import ctypes as C
import torch.distributed as dist
import gpurs_b200 as G
from gpurs_b200 import _ffi
from gpurs_b200.sharding import allgather_objects, broadcast_from_rank0
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
# what Communicator does before it touches a GPU: rank 0 makes the id through the C ABI, every rank receives the same bytes
unique = broadcast_from_rank0(dist)(G.comm_unique_id() if rank == 0 else None)
everyone = allgather_objects(dist)(unique)
ok = len(unique) == _ffi.COMM_ID_BYTES and everyone[0] == everyone[1] == unique and any(unique)
other = broadcast_from_rank0(dist)(G.comm_unique_id() if rank == 0 else None)
ok = ok and other != unique                                    # every id is fresh
library = _ffi.load()
handle = C.c_void_p()
raw = (C.c_uint8 * _ffi.COMM_ID_BYTES).from_buffer_copy(unique)
ok = ok and library.gpurs_comm_init(None, raw, 2, rank, C.byref(handle)) == _ffi.E_INVALID_ARGUMENT and not handle.value
ok = ok and library.gpurs_comm_allgather(None, None, 0, 0) == _ffi.E_INVALID_ARGUMENT
dist.barrier(); dist.destroy_process_group()
sys.exit(0 if ok else 1)
"""


def test_two_rank_gloo_communicator_id_exchange(tmp_path):
    """The host half of the NCCL all-gather, on CPU: the id is made by one rank through the C ABI (no GPU is needed for
    that), reaches the other through a gloo group, and the calls that need a GPU refuse null handles."""
    script = tmp_path / "comm_worker.py"
    script.write_text(COMM_WORKER)
    port = str(29950 + os.getpid() % 40)
    workers = [subprocess.Popen([sys.executable, str(script), str(ROOT), port, str(rank)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
               for rank in range(2)]
    for worker in workers:
        output, _ = worker.communicate(timeout=240)
        assert worker.returncode == 0, output.decode()[-2000:]
