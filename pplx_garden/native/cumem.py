"""CUDA virtual-memory-management helpers: allocations that can be exported to other processes
as POSIX file descriptors, imported, mapped at chosen addresses, and bound to NVLink multicast
objects. The classes are implemented in csrc/cumem/cumem.{h,cpp} and bound in
csrc/bindings/py_cumem.cpp; this module gives them their public import path (the one the
reference uses for its Rust classes, python/pplx_garden/native/cumem.py:3-11) and the stub
beside it (cumem.pyi) carries their signatures."""

from pplx_garden import _native as _n

__all__ = [
    "CUAllocHandle",            # base of everything that can be mapped
    "CUMemAllocHandle",         # an allocation made by this process
    "CUMemExportHandle",        # its picklable description (pid, fd, size, granularity)
    "CUMemHandleKind",          # Local / FileDescriptor / Fabric
    "CUMemImportHandle",        # another process's allocation, opened here
    "CUMemMapping",             # a mapped address range
    "CUMulticastExportHandle",  # the same for multicast objects
    "CUMulticastHandle",
]

for _name in __all__:
    globals()[_name] = getattr(_n, _name)
del _name
