"""Python face of the runtime's device-memory plumbing: growable device buffers with a stable address (VMM), pinned
staging buffers and the threaded file -> device loader.  Reference: engine-rs/src/kv_pool.rs:53-241 (VMM backend),
shim/vmm.cpp, shim/host_pin.cuh, weights.rs:194-283."""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import runtime as rt


class _CudaView:
    """Exposes a raw device range to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


class GrowableDeviceBuffer:
    """A device byte buffer that grows and shrinks in place: tensors made from it keep their address, bytes past the
    backed size are unmapped (touching them faults, so `view` only hands out backed ranges)."""

    def __init__(self, device: int, max_bytes: int, fake: bool = False):
        self.region = rt.rt().VmmRegion(device, max_bytes, fake)
        self.device, self.fake = device, fake

    @property
    def size(self) -> int:
        return self.region.size

    def resize(self, nbytes: int) -> int:
        return self.region.resize(nbytes)

    def view_unchecked(self, nbytes: int) -> torch.Tensor:
        """uint8 tensor over the first `nbytes` of the RESERVED range, backed or not: the caller guarantees that nothing
        touches bytes past `size` (they are unmapped).  For tensors that must keep one address while the backing grows."""
        if self.fake:
            import ctypes
            import numpy as np
            return torch.from_numpy(np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(self.region.ptr)))
        return torch.as_tensor(_CudaView(self.region.ptr, nbytes, self.region), device=f"cuda:{self.device}")

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = int(torch.tensor(shape).prod()) * torch.empty((), dtype=dtype).element_size()
        if offset + n > self.region.size:
            raise ValueError("view past the backed size of the buffer")
        if self.fake:
            import ctypes
            import numpy as np
            a = np.ctypeslib.as_array((ctypes.c_uint8 * n).from_address(self.region.ptr + offset))
            return torch.from_numpy(a).view(dtype).view(*shape)
        raw = torch.as_tensor(_CudaView(self.region.ptr + offset, n, self.region), device=f"cuda:{self.device}")
        return raw.view(dtype).view(*shape)


def load_file_range_to(t: torch.Tensor, path: str, offset: int, chunk: int = 64 << 20, n_buffers: int = 3,
                       n_threads: int = 2, direct: Optional[bool] = None):
    """Fill the contiguous device tensor `t` with file bytes [offset, offset + t.nbytes) through pinned staging buffers
    (reader threads overlap the disk reads with the host-to-device copies).  `direct` (default: SPARK_LOAD_DIRECT=1)
    reads with O_DIRECT, bypassing the page cache; the returned stats say whether the file system took the flag."""
    assert t.is_contiguous()
    if direct is None:
        direct = os.environ.get("SPARK_LOAD_DIRECT", "0") == "1"
    n = t.numel() * t.element_size()
    if t.is_cuda:
        with torch.cuda.device(t.device):
            return rt.rt().fast_load(path, offset, n, t.data_ptr(), torch.cuda.current_stream().cuda_stream, chunk,
                                      n_buffers, n_threads, False, bool(direct))
    return rt.rt().fast_load(path, offset, n, t.data_ptr(), 0, chunk, n_buffers, n_threads, True, bool(direct))
