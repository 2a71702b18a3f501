"""Host-side multi-GPU logic on CPU: two gloo ranks run the sharding plans, assemble a column-block
sharded integer product and a unit-sharded row set with the library's gather helpers, and take the
max-over-ranks time.  The per-rank compute here is numpy (the CUDA kernels need a GPU); what is under
test is the partitioning, the gather layout and the timing reduction."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from catena_lang_b200 import shard
    rng = np.random.default_rng(4)
    m, n, k = 48, 1000, 64
    a = rng.integers(-128, 128, (m, k)).astype(np.int64)
    bt = rng.integers(-128, 128, (n, k)).astype(np.int64)
    blocks = shard.column_blocks(n, world, align=256)
    mine = blocks[rank]
    local = torch.from_numpy(a @ bt[mine.n0:mine.n1].T)
    full = shard.gather_columns(local, blocks, m, dist)
    assert torch.equal(full, torch.from_numpy(a @ bt.T))
    for mm in (1024, 700):                                  # equal blocks (one collective) and ragged blocks
        a2 = rng.integers(-128, 128, (mm, k)).astype(np.int64)
        rblocks = shard.row_blocks(mm, world, align=256)
        mine_r = rblocks[rank]
        local_r = torch.from_numpy(a2[mine_r.m0:mine_r.m1] @ bt.T)
        full_r = shard.gather_rows(local_r, rblocks, dist)
        assert torch.equal(full_r, torch.from_numpy(a2 @ bt.T))
    units, width = 37, 16
    rows = torch.arange(units * width, dtype=torch.float32).reshape(units, width)
    ranges = shard.unit_ranges(units, world)
    got = shard.gather_units(rows[ranges[rank].u0:ranges[rank].u1].clone(), ranges, width, dist)
    assert torch.equal(got, rows)
    # a map sharded by index ranges: every rank produces its range of out[i] = f(i), the gather puts them in order
    total = 1001
    iranges = shard.index_ranges(total, world, align=4)
    mine_i = iranges[rank]
    local_i = (torch.arange(mine_i.i0, mine_i.i1, dtype=torch.float32) * 3 + 1).reshape(-1, 1)
    got_i = shard.gather_units(local_i, iranges, 1, dist)
    assert torch.equal(got_i.reshape(-1), torch.arange(total, dtype=torch.float32) * 3 + 1)
    worst = shard.max_over_ranks(1.0 + rank, dist)
    assert worst == float(world)
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").close()


def test_plans_are_tile_aligned_and_cover():
    sys.path.insert(0, ROOT)
    from catena_lang_b200 import shard
    for n in (4096, 16384, 1000, 256, 1):
        for world in (1, 2, 4, 8):
            blocks = shard.column_blocks(n, world)
            assert blocks[0].n0 == 0 and blocks[-1].n1 == n
            for x, y in zip(blocks, blocks[1:]):
                assert x.n1 == y.n0 and x.n1 % 256 == 0 or x.n1 == n
            rows = shard.row_blocks(n, world)
            assert rows[0].m0 == 0 and rows[-1].m1 == n
            assert all(x.m1 == y.m0 and (x.m1 % 256 == 0 or x.m1 == n) for x, y in zip(rows, rows[1:]))
            idx = shard.index_ranges(n, world, align=4)
            assert idx[0].i0 == 0 and idx[-1].i1 == n and all(x.i1 == y.i0 and (x.i1 % 4 == 0 or x.i1 == n) for x, y in zip(idx, idx[1:]))
            ranges = shard.unit_ranges(256, world)
            assert ranges[0].u0 == 0 and ranges[-1].u1 == 256
            assert all(x.u1 == y.u0 for x, y in zip(ranges, ranges[1:]))


@pytest.mark.timeout(120)
def test_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
