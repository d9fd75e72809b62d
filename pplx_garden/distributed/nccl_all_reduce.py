"""All-reduce through a torch.distributed process group (NCCL on GPUs: NVLink 5 / NVLS on
an NVSwitch box; Gloo in CPU-only runs). Counterpart of the reference's
python/pplx_garden/distributed/nccl_all_reduce.py:12-68."""

from __future__ import annotations

from contextlib import contextmanager
from typing import Iterator, Optional

import torch
import torch.distributed as dist
from torch.distributed import ReduceOp

from pplx_garden.distributed.distributed_ops import Reducer, ReducerBuilder


class NcclReducer(Reducer):
    def __init__(self, group: dist.ProcessGroup, op: ReduceOp.RedOpType = ReduceOp.SUM) -> None:
        self._group = group
        self._op = op

    @property
    def input(self) -> Optional[torch.Tensor]:
        return None  # the collective works in place on the caller's tensor

    def reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        target = x if out is None else out
        if target is not x:
            target.copy_(x)
        dist.all_reduce(target, op=self._op, group=self._group)
        return target


class NcclAllReduce(ReducerBuilder):
    def __init__(self, group: dist.ProcessGroup) -> None:
        self._group = group

    def reducer(self, shape: torch.Size, dtype: torch.dtype,
                op: ReduceOp.RedOpType = ReduceOp.SUM) -> Reducer:
        return NcclReducer(self._group, op)

    def all_reduce(self, x: torch.Tensor, op: ReduceOp.RedOpType = ReduceOp.SUM) -> torch.Tensor:
        dist.all_reduce(x, op=op, group=self._group)
        return x

    def destroy(self) -> None:
        pass

    @contextmanager
    def capture(self) -> Iterator[None]:
        # NCCL collectives are graph-capturable as they are.
        yield
