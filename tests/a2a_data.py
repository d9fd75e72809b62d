"""Deterministic per-rank inputs for the all-to-all tests (same recipe as the reference's
tests/p2p_all_to_all/data.py:9-108: seed = dp-group index, |N(0,1)|+1 scores -> top-k,
weights normalised to sum 1 so that combine(f(x)) == f(x) for a row-wise f)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class RankData:
    indices: torch.Tensor
    weights: torch.Tensor
    dp_x: torch.Tensor
    dp_x_scale: Optional[torch.Tensor]
    expected_num_tokens: torch.Tensor  # int32 [num_experts], routes of this group only


def make_rank_data(*, seed: int, num_experts: int, topk: int, num_tokens: int, hidden_dim: int,
                   hidden_dim_scale: Optional[int], in_dtype: torch.dtype,
                   device: torch.device) -> RankData:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    scores = torch.randn((num_tokens, num_experts), generator=gen).abs() + 1
    indices = torch.topk(scores, topk, dim=-1).indices
    counts = torch.bincount(indices.flatten(), minlength=num_experts).to(torch.int32)
    x = torch.randn((num_tokens, hidden_dim), generator=gen)
    scale = None
    if hidden_dim_scale is not None:
        scale = torch.randn((num_tokens, hidden_dim_scale), generator=gen)
    weights = torch.rand((num_tokens, topk), generator=gen)
    weights = weights / weights.sum(dim=-1, keepdim=True)
    return RankData(
        indices=indices.to(torch.uint32).to(device),
        weights=weights.to(device),
        dp_x=x.to(in_dtype).to(device),
        dp_x_scale=None if scale is None else scale.to(device),
        expected_num_tokens=counts,
    )


def act(x: torch.Tensor, x_scale: Optional[torch.Tensor]) -> torch.Tensor:
    """The stand-in expert: 2x (after de-quantising when scales are present)."""
    if x_scale is None:
        return x * 2
    rep = x.shape[1] // x_scale.shape[1]
    return x.to(torch.float32) * x_scale.repeat_interleave(rep, dim=1) * 2
