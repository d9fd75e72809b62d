"""Abstract view of "the ranks I communicate with".

The concrete implementation is :class:`pplx_garden.distributed.torch_group.TorchParallelGroup`.
Method set and semantics follow the reference's
python/pplx_garden/distributed/parallel_group.py:18-143.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from contextlib import contextmanager
from typing import Iterator, TypeVar

import torch
from torch.distributed import ReduceOp, Work

from pplx_garden.distributed.distributed_ops import Reducer

T = TypeVar("T")


class ParallelGroup(ABC):
    # ---- identity ----
    @property
    @abstractmethod
    def device(self) -> torch.device:
        """Device of this rank (a CUDA device, or CPU in host-only runs)."""

    @property
    @abstractmethod
    def rank(self) -> int:
        """Index of this process inside the group."""

    @property
    @abstractmethod
    def global_rank(self) -> int:
        """Index of this process in the world."""

    @property
    @abstractmethod
    def node_rank(self) -> int:
        """Index of the node this process runs on."""

    @property
    @abstractmethod
    def local_rank(self) -> int:
        """Index of this process on its node."""

    @property
    @abstractmethod
    def size(self) -> int:
        """Number of processes in the group."""

    @property
    @abstractmethod
    def is_inter_node(self) -> bool:
        """True when the group cannot fit one NVLink domain."""

    @property
    def has_nvshmem(self) -> bool:
        return False

    # ---- CPU-side (Gloo) ----
    @abstractmethod
    def broadcast_object(self, obj: T | None, root: int) -> T: ...

    @abstractmethod
    def broadcast_cpu_tensor_async(self, tensor: torch.Tensor, root: int) -> Work: ...

    @abstractmethod
    def all_gather_object(self, obj: T) -> list[T]: ...

    @abstractmethod
    def all_reduce_cpu_async(self, x: torch.Tensor, op: ReduceOp.RedOpType = ReduceOp.SUM) -> Work: ...

    def all_reduce_cpu(self, x: torch.Tensor, op: ReduceOp.RedOpType = ReduceOp.SUM) -> None:
        self.all_reduce_cpu_async(x, op).wait()

    # ---- device-side (NCCL) ----
    @abstractmethod
    def reducer(self, shape: torch.Size, dtype: torch.dtype,
                op: ReduceOp.RedOpType = ReduceOp.SUM) -> Reducer: ...

    @abstractmethod
    def all_reduce(self, x: torch.Tensor, op: ReduceOp.RedOpType = ReduceOp.SUM) -> torch.Tensor: ...

    @abstractmethod
    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor: ...

    @abstractmethod
    def broadcast(self, tensor: torch.Tensor, root: int) -> torch.Tensor: ...

    @abstractmethod
    def all_to_all(self, tensor: torch.Tensor) -> torch.Tensor:
        """``tensor[j]`` goes to rank j; the result's slice j came from rank j."""

    @abstractmethod
    def barrier(self) -> None: ...

    @abstractmethod
    @contextmanager
    def capture(self) -> Iterator[None]:
        """Context under which the group's collectives may be captured in a CUDA graph."""

    @abstractmethod
    def destroy(self) -> None: ...

    # ---- sub-groups ----
    @abstractmethod
    def slice_by_count(self, slice_count: int) -> "ParallelGroup":
        """Split into ``slice_count`` equal consecutive groups; return the one holding this rank."""

    @abstractmethod
    def slice_by_lens(self, slice_lens: list[int]) -> "ParallelGroup":
        """Split into consecutive groups of the given sizes (which must add up to ``size``)."""
