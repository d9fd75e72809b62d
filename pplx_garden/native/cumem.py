"""CUDA virtual-memory-management helpers (see csrc/cumem/cumem.h).
Same names as the reference's python/pplx_garden/native/cumem.py:3-11."""

from pplx_garden._native import (
    CUAllocHandle as CUAllocHandle,
    CUMemAllocHandle as CUMemAllocHandle,
    CUMemExportHandle as CUMemExportHandle,
    CUMemHandleKind as CUMemHandleKind,
    CUMemImportHandle as CUMemImportHandle,
    CUMemMapping as CUMemMapping,
    CUMulticastExportHandle as CUMulticastExportHandle,
    CUMulticastHandle as CUMulticastHandle,
)
