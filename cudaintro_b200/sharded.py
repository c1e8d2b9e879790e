"""Row-sharded GEMM over several GPUs: one process per GPU, rows of A split across the ranks, B
(and the per-column scales) replicated, every rank computes its slab of C at its final position
inside a full-size buffer, and one in-place all-gather completes C on every rank.

The partition and the gather are plain ``torch.distributed`` (NCCL on GPUs; the tests run the
same code over gloo on CPU ranks with a stand-in for the slab computation).  The slab itself is
computed by the C-ABI GEMM entry points (see :func:`gemm_slab`).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class RowPartition:
    """Rows [row0, row0 + rows) of an M-row matrix belong to `rank`; every rank's slot in the
    gathered buffer is `slot_rows` tall (the last ranks may own fewer, or no, real rows)."""

    M: int
    world: int
    rank: int
    slot_rows: int
    row0: int
    rows: int

    @property
    def padded_rows(self) -> int:
        return self.slot_rows * self.world


def partition_rows(M: int, world: int, rank: int) -> RowPartition:
    if M <= 0 or world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad partition request M={M} world={world} rank={rank}")
    slot = -(-M // world)
    row0 = min(M, rank * slot)
    rows = max(0, min(M, (rank + 1) * slot) - row0)
    return RowPartition(M, world, rank, slot, row0, rows)


class ShardedGemm:
    """Owns the full C buffer of one rank and runs `compute slab -> all-gather` steps.

    ``compute_slab(c_slab)`` must fill ``c_slab`` (a view of this rank's rows of C) and may be
    asynchronous on the current stream; on GPUs it is one GEMM launch.
    """

    def __init__(self, M: int, N: int, out_dtype, device, group=None):
        import torch
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.part = partition_rows(M, self.world, self.rank)
        self.N = N
        self.c_full = torch.empty((self.part.padded_rows, N), dtype=out_dtype, device=device)
        r0 = self.rank * self.part.slot_rows
        self.c_slot = self.c_full[r0:r0 + self.part.slot_rows]     # what the all-gather sends
        self.c_slab = self.c_slot[: self.part.rows]                # the rows this rank really owns

    def gather(self):
        if self.world > 1:
            self.dist.all_gather_into_tensor(self.c_full, self.c_slot, group=self.group)

    def step(self, compute_slab):
        if self.part.rows > 0:
            compute_slab(self.c_slab)
        self.gather()

    def result(self):
        """The assembled C, [M, N] (a view without the padding rows)."""
        return self.c_full[: self.part.M]


def gemm_slab(kind: str, a, b, c_slab, row_scale=None, col_scale=None):
    """One GEMM launch for this rank's rows: `kind` in {"bf16", "f16", "i8", "w8a8"}."""
    from . import capi

    if kind == "bf16":
        capi.gemm_bf16(a, b, out=c_slab)
    elif kind == "f16":
        capi.gemm_f16(a, b, out=c_slab)
    elif kind == "i8":
        capi.gemm_i8_i32(a, b, out=c_slab)
    elif kind == "w8a8":
        capi.gemm_w8a8_bf16(a, b, row_scale, col_scale, out=c_slab)
    else:
        raise ValueError(f"unknown kind {kind!r}")


class _RawDeviceBytes:
    """Lets torch wrap device memory it did not allocate (the CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerBuffer:
    """`nbytes` of device memory on every rank, allocated by the library (``b200_peer_alloc``),
    exported with CUDA IPC and mapped by all other ranks: ``ptrs[g]`` is rank g's buffer as seen
    from this process, ``local`` a torch uint8 view of this rank's own."""

    def __init__(self, nbytes: int, device, group=None):
        import ctypes as C

        import torch
        import torch.distributed as dist

        from . import capi

        self.capi, self.dist, self.group = capi, dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = nbytes
        with torch.cuda.device(device):
            ptr = C.c_void_p()
            capi._check(capi.lib.b200_peer_alloc(nbytes, C.byref(ptr)))
            self._local_ptr = ptr.value
            handle = C.create_string_buffer(64)
            capi._check(capi.lib.b200_ipc_export(ptr, handle))
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, handle.raw, group=group)
            self._imported, self.ptrs = [], []
            for r in range(self.world):
                if r == self.rank:
                    self.ptrs.append(self._local_ptr)
                else:
                    p = C.c_void_p()
                    capi._check(capi.lib.b200_ipc_import(handles[r], C.byref(p)))
                    self._imported.append(p.value)
                    self.ptrs.append(p.value)
        self.local = torch.as_tensor(_RawDeviceBytes(self._local_ptr, nbytes), device=device)

    def close(self):
        for p in self._imported:
            self.capi.lib.b200_ipc_close(p)
        self._imported = []
        if self._local_ptr:
            self.local = None
            self.capi.lib.b200_peer_free(self._local_ptr)
            self._local_ptr = None


class SymmetricBuffer:
    """`nbytes` of device memory on every rank from torch's symmetric-memory allocator, mapped by all
    ranks: ``ptrs[g]`` is rank g's buffer as seen from this process, ``local`` a torch uint8 view of this
    rank's own, and ``mc_ptr`` a multicast address of the whole group (0 when the GPUs or the driver
    offer no NVLink multicast): a ``multimem`` store to ``mc_ptr + off`` lands at ``off`` in every
    rank's buffer.  Same interface as :class:`PeerBuffer`; torch only allocates and maps here."""

    def __init__(self, nbytes: int, device, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = nbytes
        self.local = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self._handle = symm.rendezvous(self.local, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
        self.mc_ptr = int(self._handle.multicast_ptr or 0)

    def close(self):
        self._handle = None
        self.local = None


class FusedShardedGemm:
    """Row-sharded GEMM whose epilogue writes each finished tile of this rank's slab into EVERY
    rank's copy of C (peer memory mapped with CUDA IPC), so the gather travels over NVLink while
    the remaining tiles are still being computed.  A step is the GEMM launch plus a one-warp
    marker kernel (``b200_peer_marker``): every rank writes the step number into a flag on each
    peer and waits, with a bound, until all ranks' flags have arrived, which tells it that every
    slab has landed in its copy of C.
    """

    def __init__(self, M: int, N: int, out_dtype, device, group=None, multicast: bool = False):
        """multicast=True: C lives in symmetric memory with an NVLink multicast mapping and every tile
        is written once with ``multimem.st`` (``b200_gemm_multicast``) instead of once per rank; raises
        RuntimeError where no multicast mapping can be had.  Not for runs in which a rank may leave."""
        import ctypes as C

        import torch

        import torch.distributed as dist

        itemsize = torch.empty((), dtype=out_dtype).element_size()

        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.part = partition_rows(M, self.world, self.rank)
        self.N = N
        self.multicast = bool(multicast) and self.world > 1
        if self.multicast:
            self._c = SymmetricBuffer(self.part.padded_rows * N * itemsize, device, group)
            if not self._c.mc_ptr:
                raise RuntimeError("no NVLink multicast mapping is available for this group")
            from . import capi as _capi

            self._c.capi = _capi
        else:
            self._c = PeerBuffer(self.part.padded_rows * N * itemsize, device, group)
        self._flags = PeerBuffer(256, device, group)
        self._flags.local.zero_()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=group)  # every rank's flags are zero before anyone signals
        self.capi = self._c.capi
        self.c_full = self._c.local.view(out_dtype).view(self.part.padded_rows, N)
        slab_offset = self.rank * self.part.slot_rows * N * itemsize
        # Destination i of this rank is rank (rank + i) % world: the kernel walks its destination list
        # from a start that rotates with CTA and tile, and with this ordering the ranks, which run in
        # step with one another, hit different receivers at any moment instead of the same one.
        self.slab_ptrs = [self._c.ptrs[(self.rank + i) % self.world] + slab_offset for i in range(self.world)]
        self.mc_slab_ptr = self._c.mc_ptr + slab_offset if self.multicast else 0
        r0 = self.rank * self.part.slot_rows
        self.c_slab = self.c_full[r0:r0 + self.part.rows]
        self._flag_ptrs = (C.c_void_p * self.world)(*[C.c_void_p(p) for p in self._flags.ptrs])
        self._step = 0

    def launch(self, what: int, a, b, row_scale=None, col_scale=None):
        """The multi-destination GEMM alone (no completion marker)."""
        if self.part.rows > 0 and self.multicast:
            self.capi.gemm_multicast(what, a, b, self.mc_slab_ptr, self.part.rows, self.N, a.shape[1], row_scale,
                                     col_scale)
        elif self.part.rows > 0:
            self.capi.gemm_multi(what, a, b, self.slab_ptrs, self.part.rows, self.N, a.shape[1], row_scale, col_scale)

    def mark(self):
        """Enqueue the cross-rank completion marker for everything launched so far."""
        if self.world > 1:
            self._step += 1
            self.capi._check(self.capi.lib.b200_peer_marker(self._flag_ptrs, self.world, self.rank, self._step,
                                                            self.capi._stream()))

    def step(self, what: int, a, b, row_scale=None, col_scale=None):
        self.launch(what, a, b, row_scale, col_scale)
        self.mark()

    def result(self):
        return self.c_full[: self.part.M]

    def close(self):
        import torch

        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier(group=self.group)
        self.c_full = None
        self.c_slab = None
        self._flags.close()
        self._c.close()
