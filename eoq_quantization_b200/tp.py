"""Row sharding of an entropy-coded linear layer over the GPUs of one node.

Every output row is an independent dot product and every tile an independent set of rANS
streams, so a layer shards by output rows with nothing to exchange while it computes: rank
r keeps only the tiles (and scales) of rows [r*N/g, (r+1)*N/g), x is replicated, and the
output slices meet once per layer in an all-gather.  No reduction is needed.

Two gathers: ``gather_rows`` (a library all-gather: NCCL over NVLink on GPUs, gloo in the CPU
tests) and ``PeerGather`` (the gather fused into the GEMV kernel: each rank stores its rows
straight into every rank's output buffer over NVLink and raises a flag; at batch 1 a library
all-gather of a few KB costs as much as the sharded kernel itself).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib


def shard_rows(n_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, equal row ranges; the row count must divide evenly so that the gather is a
    plain all-gather of equal slices."""
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def gather_rows(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """local: (..., N/g) slice of this rank -> (..., N) on every rank, slices in rank order."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local
    flat = local.reshape(-1, local.shape[-1]).contiguous()
    out = torch.empty((world * flat.shape[0], flat.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, flat, group=group)            # rank-major concatenation along dim 0
    out = out.view(world, flat.shape[0], flat.shape[1])
    if flat.shape[0] == 1:
        return out.reshape(*local.shape[:-1], world * local.shape[-1])
    return out.permute(1, 0, 2).reshape(*local.shape[:-1], world * local.shape[-1])


class RowShardedLinear:
    """One rank's share of y = x W^T: a local weight (anything with ``gemv(x) -> (..., N/g)``)
    plus the layer-boundary all-gather."""

    def __init__(self, local_weight, n_rows: int, group: Optional[dist.ProcessGroup] = None):
        self.local = local_weight
        self.n_rows = n_rows
        self.group = group

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        return self.local.gemv(x)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return gather_rows(self.local.gemv(x), self.group)


class PeerGather:
    """Output buffers shared by the ranks of one node for the fused GEMV + all-gather
    (``eoq_b200_gemv_gather``).  One process per GPU; the 64-byte CUDA IPC handles travel
    through ``torch.distributed``.

    ``gemv(weight, x, n_total, slot)`` returns this rank's view of the full ``(rows, n_total)``
    result once every rank's slice has arrived (the kernel that computes this rank's rows also
    waits for the others' on the current stream, so the call itself does not block).  Consecutive calls must use different slots and all ranks
    must make the same calls in the same order.
    """

    def __init__(self, slot_bytes: int, slots: int = 2, group: Optional[dist.ProcessGroup] = None):
        if not dist.is_initialized():
            raise RuntimeError("PeerGather needs an initialised process group")
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.slots = slots
        self.slot_bytes = slot_bytes
        self._views = {}
        lib = _lib.lib()
        handle = (C.c_ubyte * 64)()
        self._h = C.c_void_p()
        _lib.check(lib.eoq_b200_gather_create(self.world, self.rank, slots, slot_bytes, C.byref(self._h), handle),
                   "eoq_b200_gather_create")
        mine = bytes(handle)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        blob = (C.c_ubyte * (64 * self.world)).from_buffer_copy(b"".join(everyone))
        _lib.check(lib.eoq_b200_gather_connect(self._h, blob), "eoq_b200_gather_connect")
        dist.barrier(group)           # nobody writes into a peer before that peer has finished setting up

    def gemv(self, weight, x: torch.Tensor, n_total: int, slot: int, row_offset: Optional[int] = None,
             bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        from .fused import _DTYPES, _stream_ptr, require_cuda
        require_cuda(x, "PeerGather.gemv")
        x2 = x.reshape(-1, weight.cols).contiguous()
        rows = x2.shape[0]
        out_dtype = out_dtype or x.dtype
        if row_offset is None:
            row_offset = self.rank * weight.rows
        b = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
        lib = _lib.lib()
        with weight._on_device(x, "PeerGather.gemv"):
            _lib.check(lib.eoq_b200_gemv_gather(weight._h, x2.data_ptr(), _DTYPES[x.dtype], rows, _DTYPES[out_dtype],
                                                b.data_ptr() if b is not None else None, self._h, slot, row_offset, n_total,
                                                _stream_ptr()), "eoq_b200_gemv_gather")
        key = (slot, rows, n_total, out_dtype)
        view = self._views.get(key)
        if view is None:                        # wrap the slot once: no pointer queries while a stream is being captured
            ptr = lib.eoq_b200_gather_buffer(self._h, slot)
            view = self._views[key] = _tensor_from_ptr(ptr, (rows, n_total), out_dtype, x.device, keepalive=None)
        return view.reshape(*x.shape[:-1], n_total)

    def check(self) -> None:
        """Raise if a gather gave up waiting for a peer (synchronises the current stream)."""
        from .fused import _stream_ptr
        _lib.check(_lib.lib().eoq_b200_gather_status(self._h, _stream_ptr()), "eoq_b200_gather_status")

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._views.clear()                 # views of the buffers must not be used after this
            _lib.lib().eoq_b200_gather_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _CudaArray:
    """Minimal __cuda_array_interface__ holder so that torch can wrap library-owned device memory."""

    def __init__(self, ptr: int, shape, typestr: str, keepalive):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3,
                                         "strides": None}
        self._keepalive = keepalive


def _tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device, keepalive=None) -> torch.Tensor:
    if dtype == torch.bfloat16:                 # the interface has no bfloat16: wrap as int16 and reinterpret
        return torch.as_tensor(_CudaArray(ptr, shape, "<i2", keepalive), device=device).view(torch.bfloat16)
    typestr = {torch.float16: "<f2", torch.float32: "<f4"}[dtype]
    return torch.as_tensor(_CudaArray(ptr, shape, typestr, keepalive), device=device)
