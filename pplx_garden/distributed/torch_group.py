"""ParallelGroup on top of torch.distributed.

Each group owns two communicators over the same ranks: a device communicator (NCCL) for
tensors on the GPU and a command communicator (Gloo) for pickled objects and CPU tensors.
In a host-only run (no CUDA, e.g. CPU tests with world_size > 1) the Gloo communicator
serves both roles. Behaviour follows the reference's
python/pplx_garden/distributed/torch_group.py:22-310.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Iterator, Optional, TypeVar, cast

import torch
import torch.distributed as dist
from torch.distributed import ReduceOp, Work

from pplx_garden.distributed.distributed_ops import Reducer
from pplx_garden.distributed.nccl_all_reduce import NcclAllReduce
from pplx_garden.distributed.parallel_group import ParallelGroup
from pplx_garden.utils.logging_utils import get_logger
from pplx_garden.utils.torch import profile_range

logger = get_logger(__name__)

T = TypeVar("T")

# One NVSwitch domain holds at most this many GPUs.
_NVLINK_DOMAIN = 8


def _new_communicators(ranks: list[int], on_gpu: bool) -> Optional[tuple[dist.ProcessGroup, dist.ProcessGroup]]:
    """Collective over the WORLD: every process must call this with the same ``ranks``.
    Returns None on processes that are not members."""
    cmd = dist.new_group(ranks=ranks, backend="gloo")
    dev = dist.new_group(ranks=ranks, backend="nccl") if on_gpu else cmd
    member = dist.get_rank() in ranks
    if not member:
        return None
    return cast(dist.ProcessGroup, dev), cast(dist.ProcessGroup, cmd)


class TorchParallelGroup(ParallelGroup):
    def __init__(self, device: torch.device, node_rank: int, local_rank: int, global_rank: int,
                 ranks: list[int]) -> None:
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised before creating a group")
        if global_rank not in ranks:
            raise ValueError(f"global rank {global_rank} is not a member of {ranks}")
        self._device = torch.device(device)
        self._on_gpu = self._device.type == "cuda"
        self._node_rank = node_rank
        self._local_rank = local_rank
        self._global_rank = global_rank
        self._ranks = list(ranks)
        self._rank = self._ranks.index(global_rank)
        comms = _new_communicators(self._ranks, self._on_gpu)
        assert comms is not None
        self._device_group, self._cmd_group = comms
        self._reducer = NcclAllReduce(self._device_group)
        self._destroyed = False

    # ---- identity ----
    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def global_rank(self) -> int:
        return self._global_rank

    @property
    def node_rank(self) -> int:
        return self._node_rank

    @property
    def local_rank(self) -> int:
        return self._local_rank

    @property
    def size(self) -> int:
        return len(self._ranks)

    @property
    def ranks(self) -> list[int]:
        """Global ranks of the members, in group order."""
        return list(self._ranks)

    @property
    def is_inter_node(self) -> bool:
        return self.size > _NVLINK_DOMAIN

    @property
    def device_group(self) -> dist.ProcessGroup:
        return self._device_group

    @property
    def cmd_group(self) -> dist.ProcessGroup:
        return self._cmd_group

    # ---- CPU side ----
    def broadcast_object(self, obj: T | None, root: int) -> T:
        self._check_root(root)
        box = [obj]
        dist.broadcast_object_list(box, src=self._ranks[root], group=self._cmd_group)
        return cast(T, box[0])

    def broadcast_cpu_tensor_async(self, tensor: torch.Tensor, root: int) -> Work:
        self._check_root(root)
        if tensor.device.type != "cpu":
            raise ValueError("broadcast_cpu_tensor_async needs a CPU tensor")
        return cast(Work, dist.broadcast(tensor, src=self._ranks[root], group=self._cmd_group, async_op=True))

    def all_gather_object(self, obj: T) -> list[T]:
        out: list = [None] * self.size
        dist.all_gather_object(out, obj, group=self._cmd_group)
        return cast(list[T], out)

    @profile_range("all_reduce_cpu_async")
    def all_reduce_cpu_async(self, x: torch.Tensor, op: ReduceOp.RedOpType = ReduceOp.SUM) -> Work:
        if x.device.type != "cpu":
            raise ValueError("all_reduce_cpu_async needs a CPU tensor")
        return cast(Work, dist.all_reduce(x, op=op, group=self._cmd_group, async_op=True))

    # ---- device side ----
    @profile_range("reducer")
    def reducer(self, shape: torch.Size, dtype: torch.dtype,
                op: ReduceOp.RedOpType = ReduceOp.SUM) -> Reducer:
        return self._reducer.reducer(shape, dtype, op)

    @profile_range("all_reduce")
    def all_reduce(self, x: torch.Tensor, op: ReduceOp.RedOpType = ReduceOp.SUM) -> torch.Tensor:
        return self._reducer.all_reduce(x, op)

    @profile_range("all_gather")
    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if not -x.dim() <= dim < x.dim():
            raise ValueError(f"dim {dim} out of range for a tensor of shape {tuple(x.shape)}")
        dim %= x.dim()
        x = x.contiguous()
        gathered = self._gather_flat(x)
        # [size, ..., d, ...] -> [..., size * d, ...]
        gathered = gathered.movedim(0, dim)
        shape = list(x.shape)
        shape[dim] *= self.size
        return gathered.reshape(shape)

    def broadcast(self, tensor: torch.Tensor, root: int) -> torch.Tensor:
        self._check_root(root)
        dist.broadcast(tensor, src=self._ranks[root], group=self._device_group)
        return tensor

    def all_to_all(self, tensor: torch.Tensor) -> torch.Tensor:
        if tensor.dim() == 0 or tensor.shape[0] != self.size:
            raise ValueError(f"Expected leading dim {tuple(tensor.shape)[:1]} to match group size {self.size}")
        tensor = tensor.contiguous()
        out = torch.empty_like(tensor)
        try:
            dist.all_to_all_single(out, tensor, group=self._device_group)
        except RuntimeError:
            if self._on_gpu:
                raise
            # Gloo builds without alltoall: gather everything and keep our column.
            out.copy_(self._gather_flat(tensor)[:, self._rank])
        return out

    def barrier(self) -> None:
        if self._on_gpu:
            dist.barrier(group=self._device_group, device_ids=[self._device.index])
        else:
            dist.barrier(group=self._device_group)

    @contextmanager
    def capture(self) -> Iterator[None]:
        with self._reducer.capture():
            yield

    def destroy(self) -> None:
        if self._destroyed:
            return
        self._destroyed = True
        self._reducer.destroy()
        if self._device_group is not self._cmd_group:
            dist.destroy_process_group(self._device_group)
        dist.destroy_process_group(self._cmd_group)

    # ---- sub-groups ----
    def slice_by_count(self, slice_count: int) -> ParallelGroup:
        if slice_count <= 0 or self.size % slice_count != 0:
            raise ValueError(f"cannot split {self.size} ranks into {slice_count} equal groups")
        return self.slice_by_lens([self.size // slice_count] * slice_count)

    def slice_by_lens(self, slice_lens: list[int]) -> ParallelGroup:
        if sum(slice_lens) != self.size or any(n <= 0 for n in slice_lens):
            raise ValueError(f"slice lengths {slice_lens} do not partition {self.size} ranks")
        # new_group is collective over the world and order-sensitive: every member of this
        # group walks all slices in the same order and keeps only its own.
        mine: Optional[TorchParallelGroup] = None
        start = 0
        for n in slice_lens:
            members = self._ranks[start:start + n]
            start += n
            if self._global_rank in members:
                mine = TorchParallelGroup(self._device, self._node_rank, self._local_rank,
                                          self._global_rank, members)
            else:
                assert _new_communicators(members, self._on_gpu) is None
        assert mine is not None
        mine.barrier()
        return mine

    def _gather_flat(self, x: torch.Tensor) -> torch.Tensor:
        """[size, *x.shape] tensor holding every rank's ``x``."""
        flat = torch.empty(self.size * x.numel(), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x.reshape(-1), group=self._device_group)
        return flat.view(self.size, *x.shape)

    def _check_root(self, root: int) -> None:
        if not 0 <= root < self.size:
            raise ValueError(f"Invalid rank {root} for group of size {self.size}")
