"""Buffers the GPUs of one node store into one another, and the flag step that closes such an exchange.

`PeerBuffer` is the host side of the one-sided N-sharded GEMM: every rank allocates an output buffer through the
library (`bsir_peer_alloc`), the ranks swap CUDA IPC handles over `torch.distributed`, and each rank ends up with the
device address of every rank's buffer.  A GEMM is then told to store its column block into all of them
(`peer_out=`), and `signal_wait()` is the barrier that says "everybody's block has landed in my buffer".  The reference's
counterpart is its put / signal wrappers over aclshmem (bishengir/lib/Template/lib/Shmem/Shmem.cpp:27-120).

One process per GPU; all ranks of the group on one node.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

import bsir


class _DevArray:
    """Just enough of __cuda_array_interface__ for torch.as_tensor to wrap a device address without a copy."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": tuple(shape), "typestr": typestr, "version": 3, "strides": None}


_TYPESTR = {torch.bfloat16: None, torch.float16: "<f2", torch.float32: "<f4", torch.int8: "|i1", torch.int32: "<i4", torch.uint8: "|u1"}


class PeerBuffer:
    def __init__(self, nbytes: int, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        L = bsir.lib()
        ptr, off = C.c_void_p(), C.c_int64()
        bsir._check(L.bsir_peer_alloc(C.c_int64(nbytes), C.byref(ptr), C.byref(off)))
        self.nbytes, self.local, self.flags_offset = nbytes, ptr.value, off.value
        handle = (C.c_ubyte * 64)()
        bsir._check(L.bsir_peer_export(ptr, handle))
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local)
                continue
            q = C.c_void_p()
            bsir._check(L.bsir_peer_open((C.c_ubyte * 64).from_buffer_copy(h), C.byref(q)))
            self.ptrs.append(q.value)
            self._opened.append(q.value)
        self._flag_arr = (C.c_void_p * self.world)(*[q + self.flags_offset for q in self.ptrs])
        self._buf_arr = (C.c_void_p * self.world)(*self.ptrs)
        self.epoch = 0
        dist.barrier(group=group)          # nobody stores into a buffer its owner has not finished setting up

    def tensor(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """This rank's buffer as a tensor (no copy)."""
        n = 1
        for s in shape:
            n *= int(s)
        size = torch.empty(0, dtype=dtype).element_size()
        if n * size > self.nbytes:
            raise ValueError("PeerBuffer.tensor: shape exceeds the buffer")
        if dtype == torch.bfloat16:          # the array interface has no bf16: wrap as int16 and reinterpret
            return torch.as_tensor(_DevArray(self.local, shape, "<i2"), device="cuda").view(torch.bfloat16)
        return torch.as_tensor(_DevArray(self.local, shape, _TYPESTR[dtype]), device="cuda")

    def block_ptrs(self, byte_offset: int) -> List[int]:
        """The address `byte_offset` into every rank's buffer (what `peer_out=` takes)."""
        return [q + byte_offset for q in self.ptrs]

    def push(self, byte_offset: int, rows: int, row_bytes: int, pitch_bytes: int) -> None:
        """Enqueue a copy of a block of this rank's buffer to the same place in every other rank's buffer."""
        bsir._check(bsir.lib().bsir_peer_push(C.c_int32(self.rank), C.c_int32(self.world), self._buf_arr, C.c_int64(byte_offset),
                                             C.c_int64(rows), C.c_int64(row_bytes), C.c_int64(pitch_bytes), bsir._stream()))

    def signal_wait(self) -> None:
        """Enqueue, on the current stream: tell every peer that this rank's stores are done, wait for theirs.  The step
        number is kept on the device (epoch 0 form), so the call may be captured in a CUDA graph and replayed."""
        bsir._check(bsir.lib().bsir_peer_signal_wait(C.c_int32(self.rank), C.c_int32(self.world), self._flag_arr,
                                                    C.c_uint32(0), bsir._stream()))

    def close(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)       # no peer may still be storing into a buffer that goes away
        L = bsir.lib()
        for q in self._opened:
            L.bsir_peer_close(C.c_void_p(q))
        self._opened = []
        if self.local:
            L.bsir_peer_free(C.c_void_p(self.local))
            self.local = 0
