"""All-gather of the column-parallel GEMM's output slices over NVLink peer memory.

One process per GPU. Every rank allocates an arena (three slice buffers of `world` slots each, one
64-bit flag and one 64-bit step counter per peer), exchanges its CUDA IPC handle through torch.distributed and
maps the peers' arenas. A step is two launches on the caller's stream: the GEMM writes this rank's
slice into its own slot, `push` stores it into every peer's slot and posts the step flag. A push
first waits (bounded) for the peers' slices of the step before the previous one, so ranks stay within
two steps of each other without any step waiting for a round trip over NVLink; `wait` (or `push(wait_now=True)`)
waits for the slices of the current step. Steps rotate over three slice buffers, so a slice is never
overwritten while a peer may still read it. No NCCL call is on the step, which makes a sequence of
steps capturable in one CUDA graph.
"""
from __future__ import annotations

from . import capi


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


NBUF = 3  # slice buffers in rotation


def arena_layout(slice_bytes: int, world: int) -> dict:
    """Byte offsets inside an arena: data[buf][slot], flags[peer], counters."""
    slot = _round_up(slice_bytes, 256)
    data = NBUF * world * slot
    flags = _round_up(data, 256)
    counters = flags + _round_up(8 * world, 256)
    done = counters + _round_up(8 * world, 256)  # completion counter of the GEMM that pushes from its epilogue
    return {"slot": slot, "flags": flags, "counters": counters, "done": done, "bytes": done + 256}


class PeerGather:
    def __init__(self, slice_bytes: int, rank: int, world: int, exchange):
        """`exchange(handle: bytes) -> list[bytes]` returns every rank's handle in rank order
        (e.g. torch.distributed.all_gather_object); it is called once."""
        if slice_bytes <= 0 or slice_bytes % 16 != 0:
            raise capi.InvalidArgument("PeerGather: the slice must be a positive multiple of 16 bytes")
        if not (2 <= world <= 8) or not (0 <= rank < world):
            raise capi.InvalidArgument("PeerGather: world must be 2..8 and rank inside it")
        self.rank, self.world, self.slice_bytes = rank, world, slice_bytes
        self.lay = arena_layout(slice_bytes, world)
        self.base, handle = capi.peer_alloc(self.lay["bytes"])
        handles = exchange(handle)
        self.peers = [self.base if p == rank else capi.peer_open(handles[p]) for p in range(world)]

    def slot(self, buf: int, owner: int, arena: int | None = None) -> int:
        """Address of rank `owner`'s slice of buffer `buf` (0..NBUF-1) in an arena (default: this rank's)."""
        base = self.base if arena is None else arena
        return base + (buf * self.world + owner) * self.lay["slot"]

    def push(self, buf: int, stream=None, wait_now: bool = False):
        """Deliver this rank's slice of buffer `buf` to every peer (after the peers' previous slices have
        arrived); with wait_now also wait for the peers' slices of this step."""
        r, w = self.rank, self.world
        dst = [0 if p == r else self.slot(buf, r, self.peers[p]) for p in range(w)]
        flag_dst = [0 if p == r else self.peers[p] + self.lay["flags"] + 8 * r for p in range(w)]
        capi.allgather_push(self.slot(buf, r), self.slice_bytes, dst, flag_dst, self.base + self.lay["flags"],
                            self.base + self.lay["counters"], r, w, wait_now, stream)

    def gemm_push(self, desc, x, M, buf: int, stream=None):
        """The sharded GEMM (stream kernel, M <= 16) writing this rank's slice of buffer `buf` into its own arena
        and into every peer's, and posting the step: GEMM and exchange in one kernel."""
        r, w = self.rank, self.world
        dst = [0 if p == r else self.slot(buf, r, self.peers[p]) for p in range(w)]
        flag_dst = [0 if p == r else self.peers[p] + self.lay["flags"] + 8 * r for p in range(w)]
        capi.gemm_push(desc, x, self.slot(buf, r), M, dst, flag_dst, self.base + self.lay["flags"],
                       self.base + self.lay["counters"], self.base + self.lay["done"], r, w, stream)

    def gemm_carry(self, desc, x, M, buf: int, prev_buf, stream=None):
        """The sharded GEMM (stream kernel, M <= 16) writing this rank's slice of buffer `buf` into its own arena
        while it delivers the slice of buffer `prev_buf` - finished by the previous step - to every peer and
        posts that step (prev_buf None: nothing to deliver). The last step's slice goes out with push()."""
        r, w = self.rank, self.world
        have = prev_buf is not None
        dst = [0 if (p == r or not have) else self.slot(prev_buf, r, self.peers[p]) for p in range(w)]
        flag_dst = [0 if p == r else self.peers[p] + self.lay["flags"] + 8 * r for p in range(w)]
        capi.gemm_carry(desc, x, self.slot(buf, r), M, self.slot(prev_buf, r) if have else None,
                        self.slice_bytes if have else 0, dst, flag_dst, self.base + self.lay["flags"],
                        self.base + self.lay["counters"], self.base + self.lay["done"], r, w, stream)

    def wait(self, stream=None):
        """Wait on the stream until every peer's slice of the last pushed step is here."""
        capi.allgather_wait(self.base + self.lay["flags"], self.base + self.lay["counters"], self.rank, self.world,
                            stream)

    def close(self):
        for p, ptr in enumerate(self.peers):
            if p != self.rank:
                capi.peer_close(ptr)
        capi.peer_free(self.base)
        self.peers = []
