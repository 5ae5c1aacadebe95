"""Page-locked host tables for features (what the reference gets from
cudaHostRegister on its shared tensors, python/npc/utils/utils.py:70-75).

A table is an anonymous mapping advised to use transparent huge pages and
then registered with CUDA. Measured on the GPU host this takes about 5 s for
51 GB where allocating pinned memory through the caching host allocator takes
about 28 s; the gather kernel reads both at the same rate.
"""
import ctypes
import mmap

import torch

_HUGE = 2 << 20
_MADV_HUGEPAGE = 14
_ALREADY_REGISTERED = 712  # cudaErrorHostMemoryAlreadyRegistered


def register(ptr: int, nbytes: int):
    err = int(torch.cuda.cudart().cudaHostRegister(ptr, nbytes, 0))
    if err not in (0, _ALREADY_REGISTERED):
        raise RuntimeError(f"cudaHostRegister of {nbytes} bytes failed with error {err}")


class _Mapping:
    """Owns one anonymous mapping and its CUDA registration; the registration is dropped before
    the mapping goes away (a registration that outlives its mapping would make a later mapping at
    the same address fail to register, and points the driver at pages that are gone)."""

    def __init__(self, mm, whole, window, start, registered):
        self.mm, self.whole, self.window, self.start, self.registered = mm, whole, window, start, registered

    def __del__(self):
        if self.registered:
            try:
                torch.cuda.cudart().cudaHostUnregister(self.start)
            except Exception:   # interpreter shutdown: the driver is gone, and so is the registration
                pass
            self.registered = False


def alloc_table(rows: int, dim: int, dtype: torch.dtype, pin: bool = True) -> torch.Tensor:
    """A [rows, dim] host tensor on 2 MiB-aligned anonymous memory, registered
    with CUDA when `pin`. The mapping lives as long as the returned tensor."""
    esz = torch.empty(0, dtype=dtype).element_size()
    nbytes = rows * dim * esz
    if nbytes == 0:
        return torch.empty((rows, dim), dtype=dtype)
    mm = mmap.mmap(-1, nbytes + _HUGE, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS)
    whole = (ctypes.c_char * (nbytes + _HUGE)).from_buffer(mm)
    base = ctypes.addressof(whole)
    start = (base + _HUGE - 1) & ~(_HUGE - 1)
    try:
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        libc.madvise(ctypes.c_void_p(start), ctypes.c_size_t(nbytes), _MADV_HUGEPAGE)  # best effort
    except OSError:
        pass
    window = (ctypes.c_char * nbytes).from_address(start)
    t = torch.frombuffer(window, dtype=torch.uint8).view(dtype).view(rows, dim)
    if pin:
        register(start, nbytes)
    t._apt_keepalive = _Mapping(mm, whole, window, start, pin)
    return t
