"""Stand-in for the one use the reference makes of `cupy` (absent from the offline image):
wrapping a raw device pointer as a non-owning uint8 array that torch.as_tensor can view through
the CUDA array interface."""
import numpy as _np

uint8 = _np.uint8


class _UnownedMemory:
    def __init__(self, ptr, size, owner=None, device_id=-1):
        self.ptr = int(ptr)
        self.size = int(size)
        self.owner = owner


class _MemoryPointer:
    def __init__(self, mem, offset=0):
        self.mem = mem
        self.ptr = mem.ptr + int(offset)


class cuda:  # noqa: N801  (mirrors the cupy.cuda namespace)
    UnownedMemory = _UnownedMemory
    MemoryPointer = _MemoryPointer


class ndarray:  # noqa: N801
    def __init__(self, shape, dtype=uint8, memptr=None):
        self.shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        self.dtype = _np.dtype(dtype)
        self._memptr = memptr

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": self.dtype.str, "data": (self._memptr.ptr, False), "version": 3,
                "strides": None}
