"""Host side of the peer all-gather on CPU: arena layout, contract checks of the C entry (rejected
before CUDA is touched) and, with gloo ranks and a fake allocator, that every rank addresses the
same slots and flag words in every arena. The device side runs in bench.py at N > 1."""
import os
import socket

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

import w4a16_dequant_gemm_b200 as w4


def test_arena_layout():
    for slice_bytes, world in ((28672, 2), (16, 8), (2 * 14336 * 16, 4)):
        lay = w4.peer.arena_layout(slice_bytes, world)
        assert lay["slot"] >= slice_bytes and lay["slot"] % 256 == 0
        assert lay["flags"] >= w4.peer.NBUF * world * lay["slot"] and lay["flags"] % 8 == 0
        assert lay["counters"] >= lay["flags"] + 8 * world and lay["counters"] % 8 == 0
        assert lay["bytes"] >= lay["counters"] + 16


def test_push_contract():
    bad = w4.InvalidArgument
    ok = dict(src=256, nbytes=64, dst=[0, 512], flag_dst=[0, 1024], flags_local=2048, counters=4096, rank=0, world=2)

    def call(**kw):
        a = dict(ok, **kw)
        w4.capi.allgather_push(a["src"], a["nbytes"], a["dst"], a["flag_dst"], a["flags_local"], a["counters"],
                               a["rank"], a["world"])
    with pytest.raises(bad):
        w4.capi.allgather_wait(2048, 4096, 0, 1)
    with pytest.raises(bad):
        w4.capi.allgather_wait(2052, 4096, 0, 2)
    with pytest.raises(bad):
        call(world=1, dst=[0], flag_dst=[0])
    with pytest.raises(bad):
        call(world=9, dst=[0] * 9, flag_dst=[0] * 9)
    with pytest.raises(bad):
        call(rank=2)
    with pytest.raises(bad):
        call(nbytes=24)
    with pytest.raises(bad):
        call(src=260)
    with pytest.raises(bad):
        call(dst=[0, 0])  # the peer's destination is missing
    with pytest.raises(bad):
        call(flag_dst=[0, 1028])
    with pytest.raises(bad):
        w4.peer.PeerGather(24, 0, 2, lambda h: [h, h])


def test_gemm_carry_contract():
    """The GEMM that carries the previous step's slice: rejected on the host before CUDA is touched."""
    bad = w4.InvalidArgument
    desc = w4.DevicePackedW(1024, 1024, 128, 8, 1, 4096, 8192, None)  # dummy addresses: never dereferenced
    ok = dict(x=256, c=512, M=4, prev=1024, prev_bytes=8192, prev_peer=[0, 2048], flag_dst=[0, 4096], flags_local=8192,
              counters=16384, done=32768, rank=0, world=2)

    def call(**kw):
        a = dict(ok, **kw)
        w4.capi.gemm_carry(desc, a["x"], a["c"], a["M"], a["prev"], a["prev_bytes"], a["prev_peer"], a["flag_dst"],
                           a["flags_local"], a["counters"], a["done"], a["rank"], a["world"])
    for kw in (dict(M=0), dict(M=17), dict(world=1, prev_peer=[0], flag_dst=[0]), dict(rank=2), dict(prev=1028),
               dict(prev_bytes=7), dict(prev_peer=[0, 0]), dict(flag_dst=[0, 4100]), dict(done=32770), dict(flags_local=8196),
               dict(prev=None), dict(x=None)):
        with pytest.raises(bad):
            call(**kw)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # fake allocator: rank r's arena "lives" at (r + 1) << 32 in its own process and is "mapped" by
    # peer p at ((r + 1) << 32) + (p + 1) << 24; the handle carries the owner's rank
    w4.capi.peer_alloc = lambda n: ((rank + 1) << 32, bytes([rank]) * 64)
    w4.capi.peer_open = lambda h: ((h[0] + 1) << 32) + ((rank + 1) << 24)
    calls = []
    w4.capi.allgather_push = lambda *a: calls.append(a)

    def exchange(handle):
        out = [None] * world
        dist.all_gather_object(out, handle)
        return out
    pg = w4.peer.PeerGather(28672, rank, world, exchange)
    pg.push(1)
    src, nbytes, dst, flag_dst, flags_local, counters, r, w, wait_now, _ = calls[0]
    assert wait_now is False
    lay = pg.lay
    assert (nbytes, r, w) == (28672, rank, world)
    assert src == pg.base + (1 * world + rank) * lay["slot"]  # buffer 1, own slot, own arena
    for p in range(world):
        if p == rank:
            assert dst[p] == 0 and flag_dst[p] == 0
            continue
        mapped = ((p + 1) << 32) + ((rank + 1) << 24)
        assert dst[p] == mapped + (1 * world + rank) * lay["slot"]   # my slot in p's arena
        assert flag_dst[p] == mapped + lay["flags"] + 8 * rank       # p's flag word for me
    assert flags_local == pg.base + lay["flags"] and counters == pg.base + lay["counters"]
    out_q.put(rank)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_addresses_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert sorted(q.get(timeout=5) for _ in range(world)) == list(range(world))
