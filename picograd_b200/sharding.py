"""Partition of the matrix-multiply path over the GPUs of one node (one process per GPU).

picograd itself is single-device (backend/cuda/cuda.c:49-55 creates one context on device 0 and
docs/gpu-plan.md:35-36 puts multi-device out of scope); this layer is new.  The path shards with
no data-path collective:

  * pg_gemm_ex: N-column shards of B and C.  Rank r holds all of A and columns
    [start_r, start_r + count_r) of B, and produces the same columns of C.  K is never split, so
    no reduction is needed.
  * pg_bmm: batch shards.

Only when a caller wants the whole C on every rank is there an exchange, in one of two forms:

  * `gather_columns`: an all-gather of the column shards (NCCL over NVLink on GPUs, gloo on CPU in the
    tests) followed by a local re-layout, because column shards are not contiguous in a row-major matrix;
  * `PeerMatrix` + `scatter_gemm`: every rank maps the other ranks' full C into its own address space once
    (CUDA IPC) and the GEMM kernel stores each finished tile of its shard into every rank's C over NVLink
    while it computes the next ones: no collective and no re-layout pass afterwards, only a barrier.
"""
import torch
import torch.distributed as dist


def column_shards(n, world, align=8):
    """[(start, count)] per rank: contiguous column ranges whose starts are multiples of `align`
    (8 columns = 16 bytes of f16/bf16, the TMA base-address rule), sizes differing by at most
    one aligned block; trailing ranks may be empty when n is small."""
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    out, start = [], 0
    for r in range(world):
        nb = base + (1 if r < extra else 0)
        count = min(nb * align, max(n - start, 0))
        out.append((start, count))
        start += count
    return out


def batch_shards(batch, world):
    """[(start, count)] per rank for pg_bmm: contiguous batch ranges, sizes differing by at most one."""
    base, extra = divmod(batch, world)
    out, start = [], 0
    for r in range(world):
        c = base + (1 if r < extra else 0)
        out.append((start, c))
        start += c
    return out


def gather_columns(c_local, n_total, group=None, align=8, out=None, staging=None, membership=None, step=0):
    """All ranks receive the full row-major [M, n_total] matrix from the column shards.
    With a `membership`, the step is announced and every rank's presence is checked on the host first: RankLeft is
    raised instead of entering a collective that a departed rank would never join.

    On the GPU: one NCCL all-gather of the shards into a [world][M][width] staging buffer (a shard narrower than
    the widest one is padded first), then the library's re-layout kernel (pg_b200_gather_relayout) writes the
    row-major matrix.  `out` and `staging` may be passed in to keep allocations out of a timed loop.
    On the CPU (gloo, used by the tests of the host logic) the re-layout is a loop of slice copies."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if membership is not None:
        membership.announce(step)
        membership.check(step)
    shards = column_shards(n_total, world, align)
    m = c_local.shape[0]
    width = max(c for _, c in shards)
    assert c_local.shape[1] == shards[rank][1], "local shard has the wrong width"
    if c_local.shape[1] == width and c_local.is_contiguous():
        send = c_local
    else:
        send = torch.zeros((m, width), dtype=c_local.dtype, device=c_local.device)
        send[:, :c_local.shape[1]] = c_local
    recv = staging if staging is not None else torch.empty((world, m, width), dtype=c_local.dtype, device=c_local.device)
    full = out if out is not None else torch.empty((m, n_total), dtype=c_local.dtype, device=c_local.device)
    if c_local.is_cuda:
        if c_local.dtype != torch.float32:
            raise TypeError("gather_columns on the GPU takes the float32 output of pg_gemm_ex")
        from . import backend as _b
        from ._lib import lib
        dist.all_gather_into_tensor(recv, send, group=group)
        _b._ready()
        _b._check(lib.pg_b200_gather_relayout(recv.data_ptr(), full.data_ptr(), world, m, width, n_total, full.stride(0)),
                  "pg_b200_gather_relayout")
        return full
    dist.all_gather(list(recv.unbind(0)), send, group=group)
    for r, (start, count) in enumerate(shards):
        if count:
            full[:, start:start + count] = recv[r, :, :count]
    return full


class RankLeft(RuntimeError):
    """A rank of the group has left (or has not reached this step in time); `ranks` lists them."""

    def __init__(self, ranks, step):
        self.ranks, self.step = list(ranks), step
        super().__init__(f"rank(s) {self.ranks} absent at step {step}")


class Membership:
    """Who is still there?  Host-side failure detection for the one place where ranks depend on each other, the
    all-gather of `gather_columns` (the products themselves need no exchange: a rank that loses a peer still owns
    valid shards).  Every rank announces each step in the process group's key-value store before it enters a
    collective and says so when it leaves; `check` returns normally when all ranks have announced the step and raises
    RankLeft — before anything is launched on the GPU — when one has left or is late.  Ranks leave between steps
    only, with none of their kernels or collectives in flight."""

    def __init__(self, store, rank, world, prefix="pg_b200/member"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def announce(self, step):
        self.store.set(f"{self.prefix}/step/{self.rank}", str(int(step)))

    def leave(self):
        self.store.set(f"{self.prefix}/left/{self.rank}", "1")

    def _get(self, key):
        # check() wraps this in its own deadline: a key that is not there yet must not block for the store's timeout
        return self.store.get(key) if self.store.check([key]) else None

    def check(self, step, timeout_s=1.0, poll_s=0.01):
        import time
        deadline = time.monotonic() + timeout_s
        missing = []
        while True:
            missing, left = [], []
            for r in range(self.world):
                if self._get(f"{self.prefix}/left/{r}") is not None:
                    left.append(r)
                    continue
                v = self._get(f"{self.prefix}/step/{r}")
                if v is None or int(v) < int(step):
                    missing.append(r)
            if left:
                raise RankLeft(left, step)
            if not missing:
                return
            if time.monotonic() >= deadline:
                raise RankLeft(missing, step)
            time.sleep(poll_s)


def row_shards(m, world):
    """[(start, count)] per rank: contiguous row ranges of A for the upload of a replicated operand."""
    return batch_shards(m, world)


class HostShardedGemm:
    """pg_gemm_ex with HOST operands on `world` GPUs: the end-to-end form of the N-column partition.

    Every rank needs all of A.  Sending all of A over PCIe once per GPU would make the host side the limit
    (world copies of A leave host memory), so each rank uploads only rows [r*M/world, (r+1)*M/world) of A and the
    ranks all-gather A over NVLink (NCCL; row blocks are contiguous, so no re-layout), while the rank's column
    shard of B is uploaded on a second stream.  Then the local product, then the C shard goes back to the host.
    Buffers are created once; call() runs one step."""

    def __init__(self, dtype, m, n, k, group=None):
        from . import backend as _b
        self._b = _b
        self.dtype, self.m, self.n, self.k = dtype, m, n, k
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if m % self.world:
            raise ValueError("M must be a multiple of the number of GPUs for the row-block upload of A")
        self.c0, self.n_loc = column_shards(n, self.world)[self.rank]
        self.r0, self.m_loc = row_shards(m, self.world)[self.rank]
        t16 = torch.float16 if dtype == _b.PG_DTYPE_F16 else torch.bfloat16
        self.a_dev = torch.empty((m, k), dtype=t16, device="cuda")
        self.b_dev = torch.empty((k, self.n_loc), dtype=t16, device="cuda")
        self.c_dev = torch.empty((m, self.n_loc), dtype=torch.float32, device="cuda")
        self.side = torch.cuda.Stream()
        self.h2d_bytes = (self.m_loc * k + k * self.n_loc) * 2
        self.d2h_bytes = m * self.n_loc * 4

    def __call__(self, a_rows_host, b_shard_host, c_shard_host):
        """a_rows_host: this rank's row block of A [m_loc, k]; b_shard_host: its column shard of B [k, n_loc];
        c_shard_host: receives its column shard of C [m, n_loc].  Pinned host tensors (16-bit data viewed as int16
        is fine).  Returns after the result is on the host."""
        cur = torch.cuda.current_stream()
        self.side.wait_stream(cur)
        with torch.cuda.stream(self.side):
            self.b_dev.view(torch.int16).copy_(b_shard_host.view(torch.int16), non_blocking=True)
        a_rows = self.a_dev[self.r0:self.r0 + self.m_loc]
        a_rows.view(torch.int16).copy_(a_rows_host.view(torch.int16), non_blocking=True)
        if self.world > 1:
            dist.all_gather_into_tensor(self.a_dev.view(torch.uint8), a_rows.view(torch.uint8), group=self.group)    # bytes: any 16-bit type
        cur.wait_stream(self.side)
        self._b.pg_gemm_ex(self.dtype, self.m, self.n_loc, self.k, self.a_dev, self.k, self.b_dev, self.n_loc,
                           self.c_dev, self.n_loc)
        c_shard_host.copy_(self.c_dev, non_blocking=True)
        cur.synchronize()


class _DeviceArray:
    """A raw device allocation as the CUDA array interface, so that torch can view it as a tensor."""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 3,
                                         "strides": None}


class PeerMatrix:
    """A row-major [rows, cols] f32 matrix per rank, each mapped into every other rank's address space (CUDA IPC
    over pg_b200_ipc_export / pg_b200_ipc_open; one process per GPU on one node).  `ptrs[r]` is rank r's matrix as
    this process addresses it (`ptrs[rank]` the local one, also available as the tensor `local`)."""

    def __init__(self, rows, cols, group=None):
        import ctypes
        from . import _lib
        from .backend import _check, _ready
        _ready()
        self._lib, self._check = _lib.lib, _check
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.rows, self.cols = rows, cols
        # an allocation of its own (cudaMalloc through the library), so that the handle names exactly this matrix.
        # A rank that cannot allocate or export still takes part in the exchange below (with no handle), so that the
        # ranks fail together instead of leaving the others waiting in a collective.
        self._opened, self.ptrs, self.local = [], [], None
        self._base = self._lib.pg_b200_malloc(rows * cols * 4)
        mine = None
        if self._base:
            self.local = torch.as_tensor(_DeviceArray(self._base, (rows, cols)), device="cuda")
            handle = (ctypes.c_ubyte * 64)()
            if self._lib.pg_b200_ipc_export(self._base, handle) == 0:
                mine = (bytes(handle), 0, torch.cuda.current_device())
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        for r, entry in enumerate(everyone):
            if entry is None or mine is None:
                self.ptrs.append(None)
                continue
            h, offset, _dev = entry
            if r == self.rank:
                self.ptrs.append(self.local.data_ptr())
                continue
            p = ctypes.c_void_p()
            if self._lib.pg_b200_ipc_open((ctypes.c_ubyte * 64).from_buffer_copy(h), ctypes.byref(p)) != 0:
                self.ptrs.append(None)
                continue
            self._opened.append(p.value)
            self.ptrs.append(p.value + offset)
        # every rank learns whether every mapping succeeded, so that all of them give up together
        good = torch.tensor([0 if None in self.ptrs else 1], device="cuda")
        dist.all_reduce(good, op=dist.ReduceOp.MIN, group=group)
        if int(good.item()) == 0:
            why = self._lib.pg_b200_last_error().decode()
            self.close()
            raise RuntimeError("a rank could not allocate, export or map a shared matrix (no peer access between these "
                               "GPUs?): " + why)

    def close(self):
        """Unmap the peers' matrices; collective (every rank must have stopped writing first)."""
        torch.cuda.synchronize()
        dist.barrier(self.group)
        for p in self._opened:
            self._check(self._lib.pg_b200_ipc_close(p), "pg_b200_ipc_close")
        self._opened = []
        dist.barrier(self.group)
        if self._base:
            self.local = None
            self._lib.pg_b200_free(self._base)
            self._base = None


def scatter_gemm(dtype, a, b_shard, peers, col0):
    """This rank's column shard C[:, col0:col0+n_loc] = a @ b_shard, stored by the GEMM kernel into the full C of every
    rank (`peers`: a PeerMatrix).  Returns without synchronising: the full C is complete on every rank after each
    rank has synchronised its stream and the ranks have met (`finish_scatter`)."""
    from .backend import pg_gemm_ex_scatter
    m, k = a.shape
    n_loc = b_shard.shape[1]
    # a chunk goes to the destinations in list order: the local matrix first, then the peers starting behind this
    # rank, so that at any moment the ranks are sending to different peers and not all to rank 0
    order = [peers.ptrs[(peers.rank + i) % peers.world] for i in range(peers.world)]
    pg_gemm_ex_scatter(dtype, m, n_loc, k, a, a.stride(0), b_shard, b_shard.stride(0), order, peers.cols, col0)


def finish_scatter(peers):
    torch.cuda.synchronize()
    dist.barrier(peers.group)
