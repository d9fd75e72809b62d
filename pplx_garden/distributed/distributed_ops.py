"""Interfaces of all-reduce providers.

A ``ReducerBuilder`` owns whatever state an all-reduce implementation needs (communicator,
registered buffers) and hands out ``Reducer`` objects bound to one shape/dtype, so that an
implementation may pre-allocate its input buffer and be captured in a CUDA graph through
``capture()``. Same contract as the reference's
python/pplx_garden/distributed/distributed_ops.py:12-56.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from contextlib import contextmanager
from typing import Iterator, Optional

import torch
from torch.distributed import ReduceOp


class Reducer(ABC):
    """An all-reduce bound to a shape, dtype and reduction op."""

    @property
    @abstractmethod
    def input(self) -> Optional[torch.Tensor]:
        """Pre-allocated tensor callers may write into to skip a copy; None if there is none."""

    @abstractmethod
    def reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Reduce ``x`` across the group; the result lands in ``out`` (default: in place)."""


class ReducerBuilder(ABC):
    @abstractmethod
    def reducer(self, shape: torch.Size, dtype: torch.dtype,
                op: ReduceOp.RedOpType = ReduceOp.SUM) -> Reducer: ...

    @abstractmethod
    def all_reduce(self, x: torch.Tensor, op: ReduceOp.RedOpType = ReduceOp.SUM) -> torch.Tensor: ...

    @abstractmethod
    def destroy(self) -> None: ...

    @contextmanager
    @abstractmethod
    def capture(self) -> Iterator[None]:
        yield
