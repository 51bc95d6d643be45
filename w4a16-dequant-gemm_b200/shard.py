"""Column-parallel sharding of the fused-dequant GEMM over the GPUs of one node.

The packed formats are row-major per output column n (a row of W), so the shard
of rank r is a contiguous slice of every array: a pointer offset and a smaller N.
Activations are replicated; the only exchange is the gather of the FP16 output
slices (NCCL over NVLink on GPUs, gloo in the CPU tests). The reference has no
multi-GPU code; this is the N-sharding its GEMM entry admits unchanged.
"""
from __future__ import annotations

from .capi import DevicePackedW, DevicePackedWm


def row_range(N: int, world: int, rank: int, align: int = 64):
    """Rows [n0, n1) of W owned by `rank`: equal shares rounded to `align` rows (the
    stream kernel's panel height), the remainder going to the last rank."""
    per = -(-N // world)
    per = -(-per // align) * align
    n0 = min(N, rank * per)
    n1 = N if rank == world - 1 else min(N, n0 + per)
    return n0, n1


def shard_w4(p: DevicePackedW, world: int, rank: int) -> DevicePackedW:
    n0, n1 = row_range(p.N, world, rank)
    wk, wg = (p.K + 7) // 8, (p.G + 7) // 8
    return DevicePackedW(n1 - n0, p.K, p.gs, p.G, p.symmetric, p.q + 4 * n0 * wk, p.scales + 2 * n0 * p.G,
                         None if p.zeros is None else p.zeros + 4 * n0 * wg)


def shard_mx(p: DevicePackedWm, world: int, rank: int) -> DevicePackedWm:
    n0, n1 = row_range(p.N, world, rank)
    return DevicePackedWm(n1 - n0, p.K, p.B, p.q + 4 * n0 * ((p.K + 7) // 8), p.scales + n0 * p.B)


def gather_columns(c_local, N: int, dist, group=None):
    """All-gather the [M, n_local] FP16 slices into the full [M, N] output on every rank.
    Shards may differ in width (last rank): slices travel padded to the widest one."""
    import torch
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    M = c_local.shape[0]
    widths = [row_range(N, world, r)[1] - row_range(N, world, r)[0] for r in range(world)]
    wmax = max(widths)
    send = c_local if c_local.shape[1] == wmax else torch.nn.functional.pad(c_local, (0, wmax - c_local.shape[1]))
    recv = torch.empty((world, M, wmax), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(recv.view(-1), send.contiguous().view(-1), group=group)
    return torch.cat([recv[r, :, :widths[r]] for r in range(world)], dim=1)
