"""N > 1 host logic on CPU: two gloo ranks shard a product by N columns (and a bmm by batch),
each computes its shard with the CPU oracle standing in for the device, and the gathered result
equals the unsharded product bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_column_shards_cover_and_align():
    from picograd_b200.sharding import batch_shards, column_shards
    for n in (1, 7, 8, 100, 8192, 14336, 4097):
        for world in (1, 2, 3, 4, 8):
            sh = column_shards(n, world)
            assert len(sh) == world
            assert sum(c for _, c in sh) == n
            pos = 0
            for s, c in sh:
                assert s == pos and (s % 8 == 0 or c == 0)
                pos += c
    assert column_shards(8192, 8) == [(i * 1024, 1024) for i in range(8)]
    assert batch_shards(64, 8) == [(i * 8, 8) for i in range(8)]
    assert [c for _, c in batch_shards(10, 4)] == [3, 3, 2, 2]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle_lib
    import workloads as wl
    from picograd_b200.sharding import batch_shards, column_shards, gather_columns
    o = oracle_lib.oracle()
    m, n, k = 48, 200, 96
    a, b = wl.config2(m, n, k)
    start, count = column_shards(n, world)[rank]
    b_loc = np.ascontiguousarray(b[:, start:start + count])
    c_loc = o.gemm_ex(wl.BF16, a, b_loc) if count else np.zeros((m, 0), np.float32)
    full = gather_columns(torch.from_numpy(c_loc), n)
    want = o.gemm_ex(wl.BF16, a, b)
    ok = bool(np.array_equal(full.numpy(), want))
    # batch shards of a bmm need no exchange at all: every rank owns whole outputs
    q, kt, _ = wl.config4(5, 16, 8)
    bs, bc = batch_shards(5, world)[rank]
    s_loc = o.bmm(wl.BF16, q[bs:bs + bc], kt[bs:bs + bc])
    ok = ok and bool(np.array_equal(s_loc, o.bmm(wl.BF16, q, kt)[bs:bs + bc]))
    open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_gloo_ranks_column_sharded_gemm(tmp_path, oracle):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"
