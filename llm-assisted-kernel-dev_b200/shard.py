"""Sharding of the two problems over the GPUs of one node.

No data-path collective is involved: the dual GEMM splits its output columns
(rows of B1/B2 and their scale-factor atoms; A and its scale factors are
replicated), the grouped GEMM assigns whole groups to ranks.  Each rank keeps
its slice of C.
"""
from __future__ import annotations


def column_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous [begin, end) output columns of ``rank``; boundaries fall on
    multiples of 128 so scale-factor atoms are never split.  The first
    ``(n/128) % world`` ranks get one extra 128-column block."""
    if n % 128:
        raise ValueError(f"n={n} is not a multiple of 128")
    blocks = n // 128
    base, extra = divmod(blocks, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * 128, end * 128


def shard_dual_input(data, rank: int, world: int):
    """View of the dual-GEMM 10-tuple restricted to this rank's output columns.
    All returned tensors alias the originals (no copies); ``c`` keeps the full
    row pitch.  Requires L == 1 (loop over batches otherwise)."""
    a, b1, b2, sfa, sfb1, sfb2, sfa_p, sfb1_p, sfb2_p, c = data
    if c.shape[2] != 1:
        raise ValueError("column sharding of a batched problem: shard each batch separately")
    n = c.shape[1]
    lo, hi = column_range(n, rank, world)
    blo, bhi = lo // 128, hi // 128
    return (a, b1[lo:hi], b2[lo:hi], sfa, sfb1[lo:hi], sfb2[lo:hi], sfa_p,
            sfb1_p[:, :, blo:bhi], sfb2_p[:, :, blo:bhi], c[:, lo:hi])


def assign_groups(problem_sizes, world: int, balance: bool = False) -> list[list[int]]:
    """Group indices owned by each rank.  Default: contiguous blocks of
    ceil(G / world) groups.  ``balance=True``: longest-processing-time greedy
    on m*n*k so ragged groups spread evenly."""
    g = len(problem_sizes)
    if not balance:
        per = (g + world - 1) // world
        return [list(range(r * per, min(g, (r + 1) * per))) for r in range(world)]
    order = sorted(range(g), key=lambda i: -(problem_sizes[i][0] * problem_sizes[i][1] * problem_sizes[i][2]))
    load = [0] * world
    owned: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = load.index(min(load))
        owned[r].append(i)
        load[r] += problem_sizes[i][0] * problem_sizes[i][1] * problem_sizes[i][2]
    return [sorted(x) for x in owned]


def shard_grouped_input(data, rank: int, world: int, balance: bool = False):
    """The grouped 4-tuple restricted to the groups this rank owns."""
    abc, sfs, sfs_perm, sizes = data
    mine = assign_groups(sizes, world, balance)[rank]
    return ([abc[i] for i in mine], [sfs[i] for i in mine], [sfs_perm[i] for i in mine], [sizes[i] for i in mine])


def gather_dual_output(c_local, n: int, group=None):
    """Optional step after a column-sharded dual GEMM: every rank ends up with the full
    ``C [M, n, L]``.  ``c_local`` is this rank's ``[M, n_local, L]`` shard (any strides).
    One ``all_gather`` over the process group (NCCL over NVLink on GPUs, gloo on CPU); the
    data path of the GEMM itself has no collective, so call this only when a consumer
    needs the whole matrix everywhere.  The reference is single-GPU and has no counterpart."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, _, l = c_local.shape
    parts = [torch.empty((m, hi - lo, l), dtype=c_local.dtype, device=c_local.device)
             for lo, hi in (column_range(n, r, world) for r in range(world))]
    dist.all_gather(parts, c_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def dual_gemm_gathered(shard_data, c_rank_ptrs, rank: int, world: int, n_total: int):
    """Column-sharded dual GEMM whose epilogue writes this rank's columns into the full
    ``C [M, n_total]`` of every rank (GEMM and all-gather of the shards in one kernel, plain
    stores over NVLink to peer-mapped buffers; ``b200_dual_gemm_nvfp4_gather``).

    shard_data   the 10-tuple of ``shard_dual_input(data, rank, world)`` (its ``c`` is not used)
    c_rank_ptrs  device addresses, as seen from this GPU, of every rank's [M, n_total] fp16 buffer
                 (this rank's own at index ``rank``; the others peer-mapped, e.g. the ``buffer_ptrs``
                 of a ``torch.distributed._symmetric_memory`` rendezvous)
    Runs on the current stream and does not synchronise; the gathered C is complete on every rank
    once all ranks' launches have finished (synchronise, then a barrier).  The reference is
    single-GPU and has no counterpart."""
    import ctypes

    import torch

    from . import _lib
    a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, _c = shard_data
    if not a.is_cuda:
        raise ValueError("dual_gemm_gathered needs CUDA tensors (there is no CPU path)")
    if len(c_rank_ptrs) != world:
        raise ValueError("one C address per rank is needed")
    m, k = a.shape[0], a.shape[1] * 2
    n_local = b1.shape[0]
    lo, hi = column_range(n_total, rank, world)
    if hi - lo != n_local:
        raise ValueError(f"the shard has {n_local} columns, rank {rank} of {world} owns {hi - lo}")
    ptrs = (ctypes.c_void_p * world)(*[int(x) for x in c_rank_ptrs])
    dev = a.device
    code = _lib.load().b200_dual_gemm_nvfp4_gather(a.data_ptr(), b1.data_ptr(), b2.data_ptr(), sfa_p.data_ptr(),
                                                   sfb1_p.data_ptr(), sfb2_p.data_ptr(), ptrs, world, rank, m, n_local,
                                                   n_total, lo, k, torch.cuda.current_stream(dev).cuda_stream, dev.index, None)
    _lib.check(code)
