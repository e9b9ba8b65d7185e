"""The multi-GPU pieces on real devices: the re-layout kernel that follows an all-gather of N-column shards (one GPU
is enough for the kernel itself), and — where the box has two GPUs — two NCCL ranks that shard a product by columns,
gather it, and run the host-operand form (row-block upload of A + all-gather of A over NVLink)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import workloads as wl

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("shape", [(4, 96, 64, 256), (3, 50, 40, 117), (8, 33, 7, 50), (2, 128, 1024, 2048)])
def test_relayout_kernel(pg, shape):
    """staging [G][rows][width] -> row-major [rows][n], n <= G * width (a ragged last shard is clipped); the padding
    columns of a wider leading dimension stay untouched."""
    g, rows, width, n = shape
    rng = np.random.default_rng(5)
    st = rng.standard_normal((g, rows, width)).astype(np.float32)
    ld = n + 4
    full = torch.full((rows, ld), 7.0, device="cuda")
    pg.pg_gather_relayout(torch.from_numpy(st).cuda(), full, g, rows, width, n)
    pg.pg_dev_sync()
    want = np.concatenate([st[i] for i in range(g)], axis=1)[:, :n]
    got = full.cpu().numpy()
    assert np.array_equal(got[:, :n], want)
    assert np.all(got[:, n:] == 7.0)


@pytest.mark.parametrize("shape", [(384, 1000, 512, 4), (1024, 2048, 1024, 8), (256, 256, 128, 1)])
def test_shard_stored_into_several_full_matrices(pg, oracle, shape):
    """pg_b200_gemm_ex_scatter on one GPU: the destinations stand in for the ranks' full C.  Every "rank" stores its
    column shard into all of them; afterwards each holds the whole product, the same bits everywhere and the same
    bits as the plain shard product, with the padding columns of a wider leading dimension untouched."""
    from picograd_b200 import sharding
    from gpu_util import to_dev
    m, n, k, world = shape
    a, b = wl.config2(m, n, k)
    ld = n + 8
    fulls = [torch.full((m, ld), 7.0, device="cuda") for _ in range(world)]
    ad = to_dev(a, wl.BF16)
    pg.set_option("k_splits", 1)          # the plain product it is compared with must not cut K either
    for rank, (c0, cnt) in enumerate(sharding.column_shards(n, world)):
        bd = to_dev(np.ascontiguousarray(b[:, c0:c0 + cnt]), wl.BF16)
        pg.pg_gemm_ex_scatter(wl.BF16, m, cnt, k, ad, k, bd, cnt, [f.data_ptr() for f in fulls], ld, c0)
        assert pg.last_path().startswith("tc:") and (world == 1 or pg.last_path().endswith(f":to{world}"))
        own = torch.empty((m, cnt), device="cuda")
        pg.pg_gemm_ex(wl.BF16, m, cnt, k, ad, k, bd, cnt, own, cnt)
        pg.pg_dev_sync()
        assert torch.equal(fulls[rank][:, c0:c0 + cnt], own)
    want = oracle.gemm_ex(wl.BF16, a, b)
    for f in fulls:
        assert torch.equal(f, fulls[0])
        got = f.cpu().numpy()
        assert wl.relerr(got[:, :n], want) <= wl.tolerance(wl.BF16, k)
        assert np.all(got[:, n:] == 7.0)


def test_scatter_refuses_what_tma_cannot_store(pg):
    a = torch.zeros((64, 64), device="cuda", dtype=torch.bfloat16)
    c = torch.zeros((64, 72), device="cuda")
    with pytest.raises(pg.PgError):                      # shard width not a multiple of 4
        pg.pg_gemm_ex_scatter(wl.BF16, 64, 62, 64, a, 64, a, 64, [c.data_ptr()], 72, 0)
    with pytest.raises(pg.PgError):                      # shard beyond the row
        pg.pg_gemm_ex_scatter(wl.BF16, 64, 64, 64, a, 64, a, 64, [c.data_ptr()], 72, 16)
    with pytest.raises(pg.PgError):                      # f32 operands
        pg.pg_gemm_ex_scatter(wl.F32, 64, 64, 64, c, 72, c, 72, [c.data_ptr()], 72, 0)
    with pytest.raises(pg.PgError):                      # nine destinations
        pg.pg_gemm_ex_scatter(wl.BF16, 64, 64, 64, a, 64, a, 64, [c.data_ptr()] * 9, 72, 0)


def test_relayout_refuses_shards_that_do_not_cover(pg):
    st = torch.zeros((2, 4, 8), device="cuda")
    full = torch.zeros((4, 32), device="cuda")
    with pytest.raises(pg.PgError):
        pg.pg_gather_relayout(st, full, 2, 4, 8, 32)


_WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path[:0] = [{root!r}, {tests!r}]
import workloads as wl, oracle_lib
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
import picograd_b200 as pg
from picograd_b200 import sharding
from gpu_util import to_dev
pg.pg_set_device(rank)
o = oracle_lib.oracle()
m, n, k = 256, 1000, 512
a, b = wl.config2(m, n, k)
c0, cnt = sharding.column_shards(n, world)[rank]
ad, bd = to_dev(a, wl.BF16), to_dev(np.ascontiguousarray(b[:, c0:c0 + cnt]), wl.BF16)
c = torch.empty((m, cnt), device="cuda")
pg.pg_gemm_ex(wl.BF16, m, cnt, k, ad, k, bd, cnt, c, cnt)
full = sharding.gather_columns(c, n)
torch.cuda.synchronize()
want = o.gemm_ex(wl.BF16, a, b)
ok = wl.relerr(full.cpu().numpy(), want) <= wl.tolerance(wl.BF16, k)
# every rank holds the same bits
ref = full.clone(); dist.broadcast(ref, 0)
ok = ok and bool(torch.equal(ref, full))
# host operands: each rank uploads its row block of A and its column shard of B, A is all-gathered over NVLink
m2, n2 = 512, 1024
a2, b2 = wl.config2(m2, n2, k)
hs = sharding.HostShardedGemm(wl.BF16, m2, n2, k)
a_rows = torch.from_numpy(np.ascontiguousarray(a2[hs.r0:hs.r0 + hs.m_loc]).view(np.int16)).pin_memory()
b_sh = torch.from_numpy(np.ascontiguousarray(b2[:, hs.c0:hs.c0 + hs.n_loc]).view(np.int16)).pin_memory()
c_sh = torch.empty((m2, hs.n_loc), dtype=torch.float32).pin_memory()
# the shard stored by the GEMM kernel itself into every rank's full C (peer memory mapped over CUDA IPC)
n3 = 1024
a3, b3 = wl.config2(m, n3, k)
c0, cnt = sharding.column_shards(n3, world)[rank]
peers = sharding.PeerMatrix(m, n3)
peers.local.fill_(-1.0)
torch.cuda.synchronize(); dist.barrier()
ad3, bd3 = to_dev(a3, wl.BF16), to_dev(np.ascontiguousarray(b3[:, c0:c0 + cnt]), wl.BF16)
sharding.scatter_gemm(wl.BF16, ad3, bd3, peers, c0)
path3 = pg.last_path()
sharding.finish_scatter(peers)
want3 = o.gemm_ex(wl.BF16, a3, b3)
ok = ok and path3.endswith(":to%d" % world)
ok = ok and wl.relerr(peers.local.cpu().numpy(), want3) <= wl.tolerance(wl.BF16, k)
c_own = torch.empty((m, cnt), device="cuda")
pg.set_option("k_splits", 1)
pg.pg_gemm_ex(wl.BF16, m, cnt, k, ad3, k, bd3, cnt, c_own, cnt)
pg.set_option("k_splits", 0)
ok = ok and bool(torch.equal(peers.local[:, c0:c0 + cnt], c_own))
ref3 = peers.local.clone(); dist.broadcast(ref3, 0)
ok = ok and bool(torch.equal(ref3, peers.local))
peers.close()
for _ in range(2):
    hs(a_rows, b_sh, c_sh)
want2 = o.gemm_ex(wl.BF16, a2, np.ascontiguousarray(b2[:, hs.c0:hs.c0 + hs.n_loc]))
ok = ok and wl.relerr(c_sh.numpy(), want2) <= wl.tolerance(wl.BF16, k)
pg.pg_dev_sync()
open(os.path.join({out!r}, f"rank{{rank}}.txt"), "w").write("ok" if ok else "mismatch")
dist.barrier(); dist.destroy_process_group()
"""


@pytest.mark.timeout(300)
def test_two_nccl_ranks_shard_gather_and_host_form(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT, tests=os.path.join(ROOT, "tests"), out=str(tmp_path)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), str(script)],
                       capture_output=True, text=True, timeout=280, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    for rank in range(2):
        assert (tmp_path / f"rank{rank}.txt").read_text() == "ok"
