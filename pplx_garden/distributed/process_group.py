"""World bootstrap and a multi-process launcher.

``ProcessGroup`` initialises torch.distributed for one rank ("cpu:gloo,cuda:nccl" on GPU
machines, Gloo only on CPU-only machines) and ``ParallelLaunch.run`` spawns one process
per device of this node and calls ``worker(device, dp_group, global_group, *args)`` in
each, returning the workers' results. ``ProcessGroup.from_env`` covers launches by
``torchrun`` / ``python -m torch.distributed.run``.

API and behaviour follow the reference's
python/pplx_garden/distributed/process_group.py:22-285 (rank 0 there runs in a spawned
child as well, despite its docstring; the results come back as pickles in a temp dir).
"""

from __future__ import annotations

import dataclasses
import datetime
import os
import pickle
import tempfile
from pathlib import Path
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pplx_garden.distributed.parallel_group import ParallelGroup
from pplx_garden.utils import logging_utils

logger = logging_utils.get_logger(__name__)


def _use_cuda(device: torch.device) -> bool:
    return torch.device(device).type == "cuda"


class ProcessGroup:
    """Owns the default (world) process group of this process."""

    def __init__(self, *, init_method: str, node_rank: int, local_rank: int, global_rank: int,
                 world_size: int, device: torch.device,
                 timeout: Optional[datetime.timedelta] = None) -> None:
        if not 0 <= global_rank < world_size:
            raise ValueError(f"global_rank {global_rank} outside [0, {world_size})")
        self._node_rank = node_rank
        self._local_rank = local_rank
        self._global_rank = global_rank
        self._world_size = world_size
        self._device = torch.device(device)
        self._owns_world = not dist.is_initialized()
        if not self._owns_world:
            if dist.get_world_size() != world_size:
                raise ValueError("an initialised world of a different size already exists")
            return
        logger.info("[rank=%d] initialising world: device=%s init_method=%s world_size=%d",
                    global_rank, self._device, init_method, world_size)
        kwargs: dict[str, Any] = dict(init_method=init_method, world_size=world_size, rank=global_rank)
        if timeout is not None:
            kwargs["timeout"] = timeout
        if _use_cuda(self._device):
            torch.cuda.set_device(self._device)
            dist.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=self._device, **kwargs)
            dist.barrier(device_ids=[self._device.index])
            torch.cuda.synchronize()
        else:
            dist.init_process_group(backend="gloo", **kwargs)
            dist.barrier()
        logger.info("[rank=%d] world ready", global_rank)

    @classmethod
    def from_env(cls, device: Optional[torch.device] = None,
                 timeout: Optional[datetime.timedelta] = None) -> "ProcessGroup":
        """Build from RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT."""
        rank = int(os.environ.get("RANK", "0"))
        local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
        if device is None:
            device = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        return cls(init_method="env://", node_rank=rank // max(local_world, 1), local_rank=local_rank,
                   global_rank=rank, world_size=world, device=device, timeout=timeout)

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def global_rank(self) -> int:
        return self._global_rank

    def create_group(self) -> ParallelGroup:
        from pplx_garden.distributed.torch_group import TorchParallelGroup

        return TorchParallelGroup(self._device, self._node_rank, self._local_rank, self._global_rank,
                                  list(range(self._world_size)))

    def destroy(self) -> None:
        if not self._owns_world or not dist.is_initialized():
            return
        if _use_cuda(self._device):
            torch.cuda.synchronize()
            dist.barrier(device_ids=[self._device.index])
        else:
            dist.barrier()
        dist.destroy_process_group()
        self._owns_world = False
        logger.info("[rank=%d] world destroyed", self._global_rank)


Worker = Callable[..., Any]


@dataclasses.dataclass
class ParallelLaunch:
    """Launch configuration.

    world_size   total number of ranks (all nodes)
    init_method  rendez-vous URL; default: a file:// URL in a temp dir (single node)
    devices      CUDA ordinals used on this node (default: the first min(#GPUs, world_size));
                 on a machine without CUDA every rank runs on the CPU
    dp_size      size of the dp group handed to the worker (consecutive ranks)
    dp_lens      alternative: explicit consecutive group sizes
    node_rank    index of this node when the job spans several
    """

    world_size: int = 1
    init_method: Optional[str] = None
    devices: Optional[list[int]] = None
    dp_size: Optional[int] = None
    dp_lens: Optional[list[int]] = None
    node_rank: int = 0
    tmpdir_base: Optional[Path] = None

    def run(self, worker: Worker, *args: Any, **kwargs: Any) -> list[Any]:
        """Run ``worker(device, dp_group, global_group, *args)`` on every local rank and
        return the list of return values (in local-rank order). With world_size == 1 the
        worker runs in this process and both groups are None."""
        if kwargs:
            raise ValueError("Keyword arguments are not supported by torch.multiprocessing.spawn()")
        if self.dp_size is not None and self.dp_lens is not None:
            raise ValueError("Cannot specify both dp_size and dp_lens")
        cuda = torch.cuda.is_available()
        devices = self.devices
        if devices is None:
            n_local = min(torch.cuda.device_count(), self.world_size) if cuda else self.world_size
            devices = list(range(n_local))
        if not devices or self.world_size % len(devices) != 0:
            raise ValueError(f"world_size {self.world_size} is not a multiple of {len(devices)} local ranks")
        num_nodes = self.world_size // len(devices)
        if not 0 <= self.node_rank < num_nodes:
            raise ValueError(f"node_rank {self.node_rank} outside [0, {num_nodes})")
        if self.dp_size is not None and (self.world_size % self.dp_size or len(devices) % self.dp_size):
            raise ValueError("dp_size must divide both the world size and the ranks per node")
        if self.dp_lens is not None and sum(self.dp_lens) != self.world_size:
            raise ValueError("dp_lens must add up to world_size")

        if self.world_size == 1:
            device = torch.device("cuda", devices[0]) if cuda else torch.device("cpu")
            return [worker(device, None, None, *args)]

        log_level = logger.getEffectiveLevel() if logging_utils.logging.getLogger().handlers else None
        with tempfile.TemporaryDirectory(dir=self.tmpdir_base) as tmp:
            tmp_path = Path(tmp)
            init_method = self.init_method
            if init_method is None:
                rendezvous = tmp_path / "rendezvous"
                rendezvous.touch()
                init_method = f"file://{rendezvous}"
            ctx = mp.start_processes(
                _child_main,
                args=(self, init_method, devices, cuda, str(tmp_path), log_level, worker, args),
                nprocs=len(devices),
                join=False,
                start_method="spawn",
            )
            while not ctx.join():
                pass
            results = []
            for local_rank in range(len(devices)):
                with open(tmp_path / f"result_{local_rank}.pkl", "rb") as f:
                    results.append(pickle.load(f))
            return results


def _child_main(local_rank: int, config: ParallelLaunch, init_method: str, devices: list[int],
                cuda: bool, tmpdir: str, log_level: Optional[int], worker: Worker,
                args: tuple) -> None:
    if log_level is not None:
        logging_utils.setup(level=log_level)
    global_rank = config.node_rank * len(devices) + local_rank
    device = torch.device("cuda", devices[local_rank]) if cuda else torch.device("cpu")
    world = ProcessGroup(init_method=init_method, node_rank=config.node_rank, local_rank=local_rank,
                         global_rank=global_rank, world_size=config.world_size, device=device)
    global_group = world.create_group()
    dp_group = global_group
    if config.dp_size is not None and config.dp_size != config.world_size:
        dp_group = global_group.slice_by_count(config.world_size // config.dp_size)
    elif config.dp_lens is not None:
        dp_group = global_group.slice_by_lens(config.dp_lens)
    try:
        result = worker(device, dp_group, global_group, *args)
    except BaseException:
        # No collective teardown on this path: the peers are not at the matching barrier, and
        # waiting for them would turn one rank's failure into a hang of the whole launch. The
        # launcher ends the other ranks as soon as this process has exited with an error.
        logger.exception("[rank=%d] worker failed", global_rank)
        raise
    with open(Path(tmpdir) / f"result_{local_rank}.pkl", "wb") as f:
        pickle.dump(result, f)
    if dp_group is not global_group:
        dp_group.destroy()
    global_group.destroy()
    world.destroy()
