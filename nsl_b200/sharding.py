"""Column-parallel sharding of a quantized linear layer over the GPUs of one node.

Only the output-feature dimension shards (rows of W[out,in], a contiguous slab of the packed
buffer: crates/nsl-runtime/src/tensor_parallel/sharding.rs:18-58 of NSL).  x and its
quantisation are replicated, so every rank's int32 accumulators equal the unsharded ones; the
one exchange step is an all-gather of the [M, N/G] outputs
(crates/nsl-runtime/src/tensor_parallel/collective.rs:1061).

Two data planes, both inside libnslq_b200.so:
  * `Comm.allgather_cols`: NCCL's all-gather, called from C++ (nslq_allgather_cols);
  * `Comm.symm_empty` + `BitLinear.forward_gathered` + `Comm.barrier`: the shards are stored
    straight into every rank's copy of the result over NVLink by the kernel that computes them.
torch.distributed is used for one thing only: handing rank 0's unique id to the other ranks
(`Comm.from_torch`); the functions at the end of the file are the torch-only mirror used by the
CPU (gloo) tests of the host logic.
"""
import ctypes as C

import torch
import torch.distributed as dist

from ._lib import check, lib
from .ops import _ptr, _stream, _tag, shard_rows

UNIQUE_ID_BYTES = 128


class _DevicePointer:
    """Lets torch wrap device memory the library allocated (CUDA array interface, version 2)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class Comm:
    """nslq_comm_t: the communicator of a column-sharded run (one process per GPU)."""

    def __init__(self, rank, world, unique_id=None):
        self.rank, self.world = rank, world
        h = C.c_void_p()
        if world > 1:
            if unique_id is None or len(unique_id) != UNIQUE_ID_BYTES:
                raise ValueError("unique_id must be the %d bytes rank 0 got from Comm.unique_id()" % UNIQUE_ID_BYTES)
            buf = C.create_string_buffer(bytes(unique_id), UNIQUE_ID_BYTES)
            check(lib().nslq_shard_init(buf, rank, world, C.byref(h)))
        else:
            check(lib().nslq_shard_init(None, 0, 1, C.byref(h)))
        self._h = h
        self._keep = []

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(UNIQUE_ID_BYTES)
        check(lib().nslq_shard_unique_id(buf))
        return buf.raw

    @classmethod
    def from_torch(cls, group=None):
        """Rank 0 mints the id and torch.distributed carries it to the others (any backend)."""
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.unique_id() if rank == 0 else None]
        if world > 1:
            dist.broadcast_object_list(box, src=0, group=group)
        return cls(rank, world, box[0])

    def close(self):
        h, self._h = self._h, None
        if h:
            lib().nslq_shard_destroy(h)

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            self.close()

    # ---- NCCL plane
    def allgather_cols(self, y_local, gathered=None, y_full=None):
        """All-gathers [M, N/G] shards.  Returns the [G, M, N/G] buffer (for M == 1 its memory
        already is y[N]); with y_full ([M, N]) the library also lays the rows out there."""
        M, n = y_local.shape
        if gathered is None:
            gathered = torch.empty(self.world, M, n, dtype=y_local.dtype, device=y_local.device)
        check(lib().nslq_allgather_cols(self._h, _ptr(y_local), _tag(y_local.dtype), M, n, _ptr(gathered),
                                        _ptr(y_full), _stream()))
        return gathered

    def wait(self, timeout_ms=0):
        check(lib().nslq_shard_wait(self._h, _stream(), int(timeout_ms)))

    # ---- peer-memory plane
    def symm_empty(self, shape, dtype):
        """A tensor in memory every rank can store into (collective: same call on every rank)."""
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        p = C.c_void_p()
        check(lib().nslq_symm_alloc(self._h, max(nbytes, 16), C.byref(p)))
        flat = torch.as_tensor(_DevicePointer(p.value, max(nbytes, 16)), device="cuda")
        return flat[:nbytes].view(dtype).view(*shape)

    def barrier(self):
        check(lib().nslq_peer_barrier(self._h, _stream()))

    def peer_allgather_cols(self, y_local, y_full):
        M, n = y_local.shape
        check(lib().nslq_peer_allgather_cols(self._h, _ptr(y_local), _tag(y_local.dtype), M, n, _ptr(y_full), _stream()))
        return y_full

    def push_cols_async(self, y_full, n_local):
        """Copy-engine form: this rank's column block of y_full ([M, world*n_local], shared) -> every peer."""
        check(lib().nslq_peer_push_cols_async(self._h, _ptr(y_full), _tag(y_full.dtype), y_full.shape[0], n_local, _stream()))

    def status(self):
        v = C.c_int()
        check(lib().nslq_shard_status(self._h, C.byref(v)))
        return v.value


# ----------------------------------------------------------------------------- torch-only mirror
def shard_weight_rows(weight_rows, world, rank):
    """Rows [row0, row0+rows) of a per-output-row tensor (packed weight, scales, zero points)."""
    r0, n = shard_rows(weight_rows.shape[0], world, rank)
    return weight_rows[r0:r0 + n].contiguous()


def gather_buffer(M, n_local, world, dtype, device):
    return torch.empty(world, M, n_local, dtype=dtype, device=device)


def all_gather_columns(y_local, gathered=None, group=None):
    """The same all-gather through torch.distributed (CPU tests with gloo).  Returns [G, M, N/G]."""
    world = dist.get_world_size(group)
    if gathered is None:
        gathered = gather_buffer(y_local.shape[0], y_local.shape[1], world, y_local.dtype, y_local.device)
    # concatenation along dim 0 of the [M, N/G] shards is exactly the [G, M, N/G] buffer
    dist.all_gather_into_tensor(gathered.view(world * y_local.shape[0], y_local.shape[1]), y_local, group=group)
    return gathered


def assemble(gathered):
    """[G, M, N/G] -> [M, N] (a view when M == 1)."""
    G, M, n = gathered.shape
    if M == 1:
        return gathered.reshape(1, G * n)
    return gathered.permute(1, 0, 2).reshape(M, G * n)
