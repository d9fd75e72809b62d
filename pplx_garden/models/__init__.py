"""Model-level building blocks on top of the kernels: the fused expert-parallel MoE layer."""

from pplx_garden.models.moe import ExpertParallelMoE as ExpertParallelMoE
from pplx_garden.models.moe import route_topk as route_topk
