"""Symmetric peer memory over NVLink for the fused compute + collective kernels.

Every rank of a process group allocates the same buffer, the CUDA IPC handles are exchanged
once over the host process group, and each rank maps all peers' buffers.  The result is a
table of device pointers (``peer_ptrs[r]`` = rank r's buffer as seen from this GPU) that the
kernels dereference directly: pull all-gather, GEMM epilogues that ``red.add`` into the
owner's gradient shard, expert dispatch/combine.  Synchronisation between ranks is a
device-side barrier on peer flags whose waits are bounded (about ``timeout_ms``); a wait that
gives up records an error in the kernel status word and the host raises on the next check.
NCCL is only used to bootstrap (handle exchange).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import lib


def _register():
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.register("ob_symm_alloc", [ctypes.POINTER(ctypes.c_void_p), L])
    lib.register("ob_symm_free", [P])
    lib.register("ob_ipc_get_handle", [P, P])
    lib.register("ob_ipc_open_handle", [P, ctypes.POINTER(ctypes.c_void_p)])
    lib.register("ob_ipc_close_handle", [P])
    lib.register("ob_ipc_handle_size", [])
    lib.register("ob_symm_barrier", [P, I, I, ctypes.c_uint, I, P, P])
    lib.register("ob_allgather_pull", [P, I, P, P, I, P])
    lib.register("ob_reduce_scatter_pull", [P, I, I, P, L, L, I, P])


_register()


class _RawCudaArray:
    """Exposes a raw device pointer through __cuda_array_interface__ so torch can wrap it."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


class PeerPtrs(list):
    """Per-rank device addresses of one symmetric region, plus the index of the local one."""

    rank = 0


class SymmetricBuffer:
    def __init__(self, nbytes: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        L = lib.load()
        p = ctypes.c_void_p()
        rc = L.ob_symm_alloc(ctypes.byref(p), self.nbytes)
        if rc:
            raise lib.KernelError(f"symmetric allocation of {self.nbytes} bytes failed ({rc})")
        self.local_ptr = p.value
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        self._opened = []
        if self.world > 1:
            hsize = L.ob_ipc_handle_size()
            buf = ctypes.create_string_buffer(hsize)
            rc = L.ob_ipc_get_handle(self.local_ptr, buf)
            if rc:
                raise lib.KernelError(f"cudaIpcGetMemHandle failed ({rc})")
            handles = [None] * self.world
            dist.all_gather_object(handles, buf.raw, group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                q = ctypes.c_void_p()
                rc = L.ob_ipc_open_handle(ctypes.create_string_buffer(h, hsize), ctypes.byref(q))
                if rc:
                    raise lib.KernelError(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
                self.peer_ptrs[r] = q.value
                self._opened.append(q.value)
        self._ptr_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        self._bytes = torch.as_tensor(_RawCudaArray(self.local_ptr, self.nbytes, self), device="cuda")

    def ptr_table(self, byte_offset: int = 0):
        """ctypes array of the peers' pointers, each advanced by ``byte_offset``."""
        if byte_offset == 0:
            return ctypes.cast(self._ptr_array, ctypes.c_void_p)
        arr = (ctypes.c_void_p * self.world)(*[p + byte_offset for p in self.peer_ptrs])
        self._last = arr
        return ctypes.cast(arr, ctypes.c_void_p)

    def peer_ptr_list(self, byte_offset: int = 0):
        out = PeerPtrs(p + byte_offset for p in self.peer_ptrs)
        out.rank = self.rank
        return out

    def view(self, dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        esz = torch.empty(0, dtype=dtype).element_size()
        return self._bytes[byte_offset:byte_offset + numel * esz].view(dtype)

    def close(self):
        L = lib.load()
        for p in self._opened:
            L.ob_ipc_close_handle(p)
        self._opened = []


class DeviceBarrier:
    """Cross-GPU barrier executed on the stream (no host synchronisation)."""

    def __init__(self, group=None, timeout_ms: int = 2000):
        self.flags = SymmetricBuffer(256, group)
        self.epoch = 0
        self.timeout_ms = timeout_ms
        self.world, self.rank = self.flags.world, self.flags.rank
        if self.world > 1:
            dist.barrier(group=group)  # every rank has mapped every flag array

    def __call__(self):
        if self.world == 1:
            return
        self.epoch += 1
        st = lib.status_tensor(torch.device("cuda", torch.cuda.current_device()))
        lib.call("ob_symm_barrier", self.flags.ptr_table(), self.world, self.rank, self.epoch, self.timeout_ms,
                 st.data_ptr(), lib.stream_ptr())


def make_copy_segments(segs, device) -> torch.Tensor:
    """segs: iterable of (src_rank, src_byte_off, dst_byte_off, nbytes) -> device table."""
    rows = []
    for r, so, do, nb in segs:
        assert so % 16 == 0 and do % 16 == 0 and nb % 16 == 0, "pull segments must be 16-byte aligned"
        rows.append([so, do, nb, r])  # CopySeg{src_off, dst_off, bytes, {src_rank, pad}}
    t = torch.tensor(rows, dtype=torch.int64)
    return t.to(device)


def allgather_pull(shard: SymmetricBuffer, dst: torch.Tensor, seg_table: torch.Tensor, shard_byte_offset: int = 0):
    lib.call("ob_allgather_pull", shard.ptr_table(shard_byte_offset), shard.world, dst.data_ptr(),
             seg_table.data_ptr(), seg_table.shape[0], lib.stream_ptr())


def reduce_scatter_pull(full: SymmetricBuffer, out: torch.Tensor, src_off_elems: int, include_self: bool = True):
    lib.call("ob_reduce_scatter_pull", full.ptr_table(), full.world, full.rank, out.data_ptr(), src_off_elems,
             out.numel(), int(include_self), lib.stream_ptr())
