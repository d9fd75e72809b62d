"""Process groups: one process per GPU, NCCL for device collectives, Gloo for CPU-side
object exchange. Public names match the reference's python/pplx_garden/distributed/__init__.py:1-7."""

from .parallel_group import ParallelGroup as ParallelGroup
from .process_group import ParallelLaunch as ParallelLaunch
from .process_group import ProcessGroup as ProcessGroup
