"""Partition of the matrix-multiply path over the GPUs of one node (one process per GPU).

picograd itself is single-device (backend/cuda/cuda.c:49-55 creates one context on device 0 and
docs/gpu-plan.md:35-36 puts multi-device out of scope); this layer is new.  The path shards with
no data-path collective:

  * pg_gemm_ex: N-column shards of B and C.  Rank r holds all of A and columns
    [start_r, start_r + count_r) of B, and produces the same columns of C.  K is never split, so
    no reduction is needed.
  * pg_bmm: batch shards.

Only when a caller wants the whole C on every rank is there an exchange: `gather_columns`, an
all-gather of the column shards (NCCL over NVLink on GPUs, gloo on CPU in the tests) followed by a
local re-layout, because column shards are not contiguous in a row-major matrix.
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


def gather_columns(c_local, n_total, group=None, align=8):
    """All ranks receive the full row-major [M, n_total] matrix from the column shards.
    Shards are padded to the widest one so that a single all_gather moves them."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shards = column_shards(n_total, world, align)
    m = c_local.shape[0]
    width = max(c for _, c in shards)
    assert c_local.shape[1] == shards[rank][1], "local shard has the wrong width"
    send = torch.zeros((m, width), dtype=c_local.dtype, device=c_local.device)
    send[:, :c_local.shape[1]] = c_local
    recv = torch.empty((world, m, width), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather(list(recv.unbind(0)), send, group=group)
    full = torch.empty((m, n_total), dtype=c_local.dtype, device=c_local.device)
    for r, (start, count) in enumerate(shards):
        if count:
            full[:, start:start + count] = recv[r, :, :count]
    return full
