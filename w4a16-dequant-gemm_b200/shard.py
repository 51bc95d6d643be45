"""Sharding of the hot path over the GPUs of one node: GEMMs column-parallel along N, decode attention across
heads (a head's K / V slab is contiguous in every array of the cache, so a shard is again a pointer offset).

The packed formats are row-major per output column n (a row of W), so the shard
of rank r is a contiguous slice of every array: a pointer offset and a smaller N.
Activations are replicated; the only exchange is the gather of the FP16 output
slices (NCCL over NVLink on GPUs, gloo in the CPU tests). The reference has no
multi-GPU code; this is the N-sharding its GEMM entry admits unchanged.
"""
from __future__ import annotations

from .capi import DeviceKVF8, DeviceKVW4, DevicePackedW, DevicePackedWm


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


def head_range(H: int, world: int, rank: int):
    """Heads [h0, h1) owned by `rank`: equal shares, the remainder spread over the first ranks."""
    base, extra = divmod(H, world)
    h0 = rank * base + min(rank, extra)
    return h0, h0 + base + (1 if rank < extra else 0)


def shard_kv_w4(p: DeviceKVW4, world: int, rank: int, slab_rows: int | None = None) -> DeviceKVW4:
    """The W4 KV cache of this rank's heads (include/w4/kvattention.cuh:39-48: H slabs per array). `slab_rows`
    is the number of rows per head slab: S for a contiguous cache (the default), npages * page for a paged pool."""
    h0, h1 = head_range(p.H, world, rank)
    rows = p.S if slab_rows is None else slab_rows
    wd, wg = (p.D + 7) // 8, (p.G + 7) // 8
    off = lambda base, per_row: None if base is None else base + h0 * rows * per_row
    return DeviceKVW4(h1 - h0, p.S, p.D, p.gs, p.G, p.symmetric, off(p.q_k, 4 * wd), off(p.s_k, 2 * p.G),
                      off(p.z_k, 4 * wg), off(p.q_v, 4 * wd), off(p.s_v, 2 * p.G), off(p.z_v, 4 * wg))


def shard_kv_f8(p: DeviceKVF8, world: int, rank: int) -> DeviceKVF8:
    """The FP8 KV cache of this rank's heads (include/w4/kvflash.cuh:390-396)."""
    h0, h1 = head_range(p.H, world, rank)
    return DeviceKVF8(h1 - h0, p.S, p.D, p.gs, p.G, p.q_k + h0 * p.S * p.D, p.s_k + 2 * h0 * p.S * p.G,
                      p.q_v + h0 * p.S * p.D, p.s_v + 2 * h0 * p.S * p.G)


def gather_heads(out_local, H: int, dist, group=None):
    """All-gather the [h_local, D] (or [nseq, h_local, D]) FP16 attention outputs into [H, D] ([nseq, H, D]) on
    every rank. Shares may differ by one head: slices travel padded to the largest one."""
    import torch
    world = dist.get_world_size(group)
    counts = [head_range(H, world, r)[1] - head_range(H, world, r)[0] for r in range(world)]
    hmax = max(counts)
    batched = out_local.dim() == 3
    x = out_local if batched else out_local.unsqueeze(0)
    if x.shape[1] < hmax:
        x = torch.nn.functional.pad(x, (0, 0, 0, hmax - x.shape[1]))
    x = x.contiguous()
    recv = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(recv.view(-1), x.view(-1), group=group)
    full = torch.cat([recv[r, :, :counts[r]] for r in range(world)], dim=1)
    return full if batched else full[0]
