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


def _leaver(rank, world, port, out_dir):
    """Three ranks; rank 2 leaves after step 0, between steps.  Ranks 0 and 1 learn of it on the host before their
    next collective (RankLeft, no hang) and go on computing their own shards, which need no exchange."""
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    import oracle_lib
    import workloads as wl
    from picograd_b200.sharding import Membership, RankLeft, column_shards, gather_columns
    store = dist.distributed_c10d._get_default_store()
    member = Membership(store, rank, world)
    o = oracle_lib.oracle()
    m, n, k = 16, 48, 32
    a, b = wl.config2(m, n, k)
    start, count = column_shards(n, world)[rank]
    c_loc = torch.from_numpy(o.gemm_ex(wl.BF16, a, np.ascontiguousarray(b[:, start:start + count])))
    verdict = []
    # step 0: everyone is there
    full = gather_columns(c_loc, n, membership=member, step=0)
    verdict.append("step0 ok" if np.array_equal(full.numpy(), o.gemm_ex(wl.BF16, a, b)) else "step0 mismatch")
    if rank == 2:
        member.leave()                      # between steps, nothing in flight
        open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("; ".join(verdict + ["left"]))
        return                              # never joins step 1 (no destroy: it is simply gone)
    try:
        gather_columns(c_loc, n, membership=member, step=1)
        verdict.append("step1 did not notice")
    except RankLeft as e:
        verdict.append(f"step1 RankLeft {e.ranks}")
    # the survivors' own work is unaffected: their shard of a new product needs no peer
    c2 = o.gemm_ex(wl.BF16, a, np.ascontiguousarray(b[:, start:start + count]))
    verdict.append("own shard ok" if np.array_equal(c2, c_loc.numpy()) else "own shard mismatch")
    open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("; ".join(verdict))


@pytest.mark.timeout(120)
def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host(tmp_path, oracle):
    world = 3
    ctx = mp.spawn(_leaver, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    import time
    deadline = time.time() + 90
    while time.time() < deadline and not all(os.path.exists(tmp_path / f"rank{r}.txt") for r in range(world)):
        time.sleep(0.2)
    texts = [open(tmp_path / f"rank{r}.txt").read() if os.path.exists(tmp_path / f"rank{r}.txt") else "no verdict" for r in range(world)]
    for p in ctx.processes:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    assert texts[2] == "step0 ok; left", texts
    for r in (0, 1):
        assert texts[r] == "step0 ok; step1 RankLeft [2]; own shard ok", texts


def test_membership_times_out_on_a_late_rank():
    from picograd_b200.sharding import Membership, RankLeft
    store = dist.HashStore()
    m0, m1 = Membership(store, 0, 2), Membership(store, 1, 2)
    m0.announce(0); m1.announce(0)
    m0.check(0)
    m0.announce(1)
    with pytest.raises(RankLeft) as e:
        m0.check(1, timeout_s=0.2)
    assert e.value.ranks == [1]
