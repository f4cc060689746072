"""Expert parallelism, host side: which experts a rank holds, and bringing the library's NCCL communicator up from a
torch.distributed process group (one process per GPU).

The reference runs one GPU per session and splits a model over cards by LAYER range only (two sessions with a host hop,
crates/shadowzero/tests/two_stage.rs:1-4); it has no expert-parallel path.  Here the experts of every MoE layer are sharded by
contiguous id range; everything else (router, attention, DeltaNet state, cache, head) is replicated, so every rank computes the
same routing and runs only the hits it holds.  The one exchange per layer is an all-reduce of the layer output in 64-bit fixed
point: integer addition is associative, so the result is bit-identical for every group size and rank order."""
import ctypes as C

import numpy as np

from . import lib as szlib

FIX_SCALE = float(1 << 40)   # one unit of the fixed-point output = 2^-40


def shard_range(rank, world, n_expert):
    """Experts [first, first + count) held by `rank`: contiguous, sizes differ by at most one, earlier ranks take the remainder."""
    if not (0 <= rank < world) or world > n_expert:
        raise ValueError(f"rank {rank} of {world} over {n_expert} experts")
    base, rem = divmod(n_expert, world)
    first = rank * base + min(rank, rem)
    return first, base + (1 if rank < rem else 0)


def owner(expert, world, n_expert):
    base, rem = divmod(n_expert, world)
    edge = rem * (base + 1)
    return expert // (base + 1) if expert < edge else rem + (expert - edge) // base


def shard_spec(rank, world, n_expert):
    """The `shard` argument of moe.MoeLayer / model.DeviceModel: rank 0 also carries the shared expert's term."""
    first, count = shard_range(rank, world, n_expert)
    return first, count, rank == 0


def to_fixed(v):
    """float64 array -> the int64 fixed-point terms the combine kernels add (round to nearest even, like cvt.rni.s64.f64)."""
    return np.rint(np.asarray(v, dtype=np.float64) * FIX_SCALE).astype(np.int64)


def from_fixed(f):
    return (np.asarray(f, dtype=np.int64).astype(np.float64) / FIX_SCALE).astype(np.float32)


def init_from_process_group(group=None, get_id=None, init=None):
    """Creates the library's communicator over the ranks of a torch.distributed group: rank 0 draws the NCCL unique id, the
    group broadcasts it (any backend), every rank joins.  `get_id` / `init` replace the library calls in host-only tests."""
    import torch
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if get_id is None or init is None:
        lib = szlib.load()

        def get_id():
            buf = (C.c_uint8 * 128)()
            szlib.check(lib.sz_ep_unique_id(buf))
            return bytes(buf)

        def init(r, w, ident):
            buf = (C.c_uint8 * 128).from_buffer_copy(ident)
            szlib.check(lib.sz_ep_init(r, w, buf))
    box = [get_id() if rank == 0 else None]
    if world > 1:
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    ident = box[0]
    assert isinstance(ident, (bytes, bytearray)) and len(ident) == 128
    init(rank, world, bytes(ident))
    return rank, world


class PeerExchange:
    """The exchange over peer memory: this rank's buffer, the peers' buffers mapped through CUDA IPC, attached to the library.
    `group`: a torch.distributed process group (one process per GPU, the current CUDA device already set).  With `group=None`
    and `local_world` set, all the ranks' buffers are allocated in this process (several ranks emulated on one GPU, for tests):
    `use(rank)` then switches the rank the library acts as."""

    def __init__(self, hidden, group=None, local_world=None):
        import torch.distributed as dist
        self.lib = szlib.load()
        self.hidden = hidden
        self.mapped = []
        n = C.c_int64()
        if local_world is not None:
            self.rank, self.world = 0, local_world
            szlib.check(self.lib.sz_ep_p2p_bytes(self.world, hidden, C.byref(n)))
            self.bufs = []
            for _ in range(self.world):
                p = C.c_uint64()
                szlib.check(self.lib.sz_ep_p2p_alloc(n.value, C.byref(p)))
                self.bufs.append(p.value)
            self.own = list(self.bufs)
            self.use(0)
            return
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        szlib.check(self.lib.sz_ep_p2p_bytes(self.world, hidden, C.byref(n)))
        p = C.c_uint64()
        szlib.check(self.lib.sz_ep_p2p_alloc(n.value, C.byref(p)))
        self.own = [p.value]
        h = (C.c_uint8 * 64)()
        szlib.check(self.lib.sz_ep_ipc_export(p.value, h))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(h), group=group)
        self.bufs = []
        for r in range(self.world):
            if r == self.rank:
                self.bufs.append(p.value)
                continue
            q = C.c_uint64()
            hb = (C.c_uint8 * 64).from_buffer_copy(handles[r])
            szlib.check(self.lib.sz_ep_ipc_import(hb, C.byref(q)))
            self.mapped.append(q.value)
            self.bufs.append(q.value)
        self.use(self.rank)
        dist.barrier(group=group)   # nobody pushes before every rank has mapped and zeroed

    def use(self, rank):
        self.rank = rank
        arr = (C.c_uint64 * self.world)(*self.bufs)
        szlib.check(self.lib.sz_ep_p2p_attach(rank, self.world, self.hidden, arr))

    def status(self):
        e = C.c_int()
        szlib.check(self.lib.sz_ep_p2p_status(C.byref(e)))
        return e.value

    def close(self):
        """Detaches, unmaps and frees.  Raises while a session that recorded passes over this exchange is alive (its CUDA graphs hold
        the buffer addresses): destroy the sessions first."""
        szlib.check(self.lib.sz_ep_p2p_detach())
        for q in self.mapped:
            szlib.check(self.lib.sz_ep_ipc_close(q))
        for p in self.own:
            szlib.check(self.lib.sz_ep_p2p_free(p))
        self.mapped, self.own = [], []
