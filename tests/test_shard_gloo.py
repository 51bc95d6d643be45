"""Multi-rank host logic on CPU (gloo, world_size 2 and 3): column-parallel row ranges,
descriptor slicing, and the gather of output slices. Each rank computes its shard with
the CPU oracle; the gathered result must equal the oracle's full GEMM bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import w4a16_dequant_gemm_b200 as w4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, K, gs, M, out_q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    o = orc.Oracle()
    p = o.quantize_w4(o.normal_f64(N * K, 3) * 0.02, N, K, gs, False)
    x = o.normal_f16(M * K, 4)
    n0, n1 = w4.shard.row_range(N, world, rank)
    # slice the packed arrays exactly as shard_w4 offsets the device pointers
    d = w4.shard.shard_w4(w4.DevicePackedW(N, K, gs, p["G"], 0, 0, 0, 0), world, rank)
    wk, wg = (K + 7) // 8, (p["G"] + 7) // 8
    assert (d.N, d.q, d.scales, d.zeros) == (n1 - n0, 4 * n0 * wk, 2 * n0 * p["G"], 4 * n0 * wg)
    ps = dict(p, N=n1 - n0, q=p["q"][d.q // 4:d.q // 4 + d.N * wk], scales=p["scales"][d.scales // 2:d.scales // 2 + d.N * p["G"]],
              zeros=p["zeros"][d.zeros // 4:d.zeros // 4 + d.N * wg])
    if n1 > n0:
        c_local = o.gemm_oracle(x, M, K, o.dequant_all_w4(ps), n1 - n0).reshape(M, n1 - n0)
    else:  # more ranks than 64-row panels: this rank owns nothing
        c_local = np.zeros((M, 0), np.float64)
    full = w4.shard.gather_columns(torch.from_numpy(c_local), N, dist)
    want = o.gemm_oracle(x, M, K, o.dequant_all_w4(p), N).reshape(M, N)
    ok = bool(np.array_equal(full.numpy(), want))
    dist.barrier()
    dist.destroy_process_group()
    out_q.put((rank, ok))


@pytest.mark.parametrize("world,N", [(2, 256), (3, 200), (2, 70)])
def test_column_parallel_gather(world, N):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, N, 96, 16, 3, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, True) for r in range(world)]


def test_row_ranges_cover_and_align():
    for N in (64, 70, 14336, 57344, 1000):
        for world in (1, 2, 4, 8):
            spans = [w4.shard.row_range(N, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == N
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(s[0] % 64 == 0 or s[0] == s[1] for s in spans)  # aligned, or an empty share


def _head_worker(rank, world, port, H, S, D, gs, out_q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    o = orc.Oracle()
    c = o.quantize_cache_w4(o.normal_f64(H * S * D, 5), o.normal_f64(H * S * D, 6), H, S, D, gs, False)
    q = o.normal_f16(H * D, 7)
    h0, h1 = w4.shard.head_range(H, world, rank)
    # slice the cache arrays exactly as shard_kv_w4 offsets the device pointers (base address 0)
    d = w4.shard.shard_kv_w4(w4.DeviceKVW4(H, S, D, gs, c["G"], 0, 0, 0, 0, 0, 0, 0), world, rank)
    wd, wg, G = (D + 7) // 8, (c["G"] + 7) // 8, c["G"]
    assert (d.H, d.q_k, d.s_k, d.z_k) == (h1 - h0, 4 * h0 * S * wd, 2 * h0 * S * G, 4 * h0 * S * wg)
    assert (d.q_v, d.s_v, d.z_v) == (d.q_k, d.s_k, d.z_k)
    nh = h1 - h0
    cs = dict(c, H=nh)
    for name, per_row, esz in (("q_k", wd, 4), ("q_v", wd, 4), ("s_k", G, 2), ("s_v", G, 2), ("z_k", wg, 4), ("z_v", wg, 4)):
        first = getattr(d, name) // esz
        cs[name] = c[name].ravel()[first:first + nh * S * per_row]
    if nh:
        out_local = o.attention_reference(q[h0 * D:h1 * D], o.dequant_cache_w4(cs, "k"), o.dequant_cache_w4(cs, "v"),
                                          nh, S, D).reshape(nh, D)
    else:
        out_local = np.zeros((0, D), np.float64)
    full = w4.shard.gather_heads(torch.from_numpy(out_local), H, dist)
    want = o.attention_reference(q, o.dequant_cache_w4(c, "k"), o.dequant_cache_w4(c, "v"), H, S, D).reshape(H, D)
    ok = bool(np.array_equal(full.numpy(), want))
    dist.barrier()
    dist.destroy_process_group()
    out_q.put((rank, ok))


@pytest.mark.parametrize("world,H", [(2, 4), (3, 5), (2, 1)])
def test_head_parallel_gather(world, H):
    """Decode attention sharded across heads: each rank runs the FP64 reference on its head slabs (sliced as
    shard_kv_w4 offsets the pointers); the gathered output equals the unsharded reference bit for bit."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_head_worker, args=(r, world, port, H, 37, 24, 8, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, True) for r in range(world)]


def test_head_ranges_cover():
    for H in (1, 8, 64, 7):
        for world in (1, 2, 4, 8):
            spans = [w4.shard.head_range(H, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == H
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
