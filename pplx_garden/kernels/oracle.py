"""Plain-PyTorch statement of what dispatch and combine must produce.

Written from the contracts (which token rows each expert receives, how they are padded,
what the weighted sum is), not from any kernel: tests compare every implementation in
this package against it, on CPU tensors and in float32.

Contract (reference: python/pplx_garden/kernels/p2p_all_to_all.py:336-359,443-517 and
tests/p2p_all_to_all/test_p2p_all_to_all.py:192-234):

* rank ``r`` owns experts ``[r * L, min((r + 1) * L, E))`` with ``L = ceil(E / world)``;
* ``out_expert_num_tokens[le]`` counts the (token, k) routes of *all dp groups* to local
  expert ``le``; a token routed twice to one expert counts twice;
* ``out_expert_x`` is expert-major, each expert's block starts at a multiple of
  ``expert_padding`` rows; the order of rows inside a block is unspecified;
* ``out_tokens[t] = sum_k weights[t, k] * expert_y[row(t, k)]`` (optionally added to the
  previous content).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


def experts_per_rank(num_experts: int, world_size: int) -> int:
    return -(-num_experts // world_size)


@dataclass
class ExpectedDispatch:
    """What one rank must hold after dispatch."""

    num_tokens: torch.Tensor            # int32 [L]
    block_start: list[int]              # first row of each local expert (padded layout)
    rows: list[torch.Tensor]            # per local expert: float32 [n, hidden] in any order
    scales: list[Optional[torch.Tensor]]  # per local expert: float32 [n, hidden_scale] or None
    total_padded_rows: int


def expected_dispatch(
    rank: int,
    world_size: int,
    num_experts: int,
    expert_padding: int,
    group_x: Sequence[torch.Tensor],
    group_x_scale: Optional[Sequence[torch.Tensor]],
    group_indices: Sequence[torch.Tensor],
    group_num_tokens: Optional[Sequence[int]] = None,
) -> ExpectedDispatch:
    """``group_*`` hold one entry per dp group (the tokens that group feeds in)."""
    L = experts_per_rank(num_experts, world_size)
    first = rank * L
    rows: list[list[torch.Tensor]] = [[] for _ in range(L)]
    scales: list[list[torch.Tensor]] = [[] for _ in range(L)]
    for g, (x, idx) in enumerate(zip(group_x, group_indices)):
        n = x.shape[0] if group_num_tokens is None else group_num_tokens[g]
        idx = idx.to(torch.int64)
        for t in range(n):
            for k in range(idx.shape[1]):
                e = int(idx[t, k])
                if first <= e < min(first + L, num_experts):
                    rows[e - first].append(x[t].to(torch.float32).cpu())
                    if group_x_scale is not None:
                        scales[e - first].append(group_x_scale[g][t].to(torch.float32).cpu())
    counts = torch.tensor([len(r) for r in rows], dtype=torch.int32)
    starts, cursor = [], 0
    for n in counts.tolist():
        starts.append(cursor)
        cursor += -(-n // expert_padding) * expert_padding
    hidden = group_x[0].shape[1]
    stacked = [torch.stack(r) if r else torch.empty((0, hidden)) for r in rows]
    if group_x_scale is not None:
        hs = group_x_scale[0].shape[1]
        stacked_scales: list[Optional[torch.Tensor]] = [
            torch.stack(s) if s else torch.empty((0, hs)) for s in scales]
    else:
        stacked_scales = [None] * L
    return ExpectedDispatch(counts, starts, stacked, stacked_scales, cursor)


def _sort_rows(m: torch.Tensor) -> torch.Tensor:
    """Rows in lexicographic order (to compare two multisets of rows)."""
    if m.shape[0] <= 1:
        return m
    order = list(range(m.shape[0]))
    keys = m.tolist()
    order.sort(key=lambda i: keys[i])
    return m[order]


def check_dispatch(
    expected: ExpectedDispatch,
    out_expert_num_tokens: torch.Tensor,
    out_expert_x: torch.Tensor,
    out_expert_x_scale: Optional[torch.Tensor],
) -> None:
    """Raise AssertionError unless the dispatch output holds exactly the expected rows."""
    got_counts = out_expert_num_tokens.cpu().to(torch.int32)
    torch.testing.assert_close(got_counts, expected.num_tokens, rtol=0, atol=0)
    x = out_expert_x.cpu().to(torch.float32)
    for le, (start, want) in enumerate(zip(expected.block_start, expected.rows)):
        n = want.shape[0]
        got = x[start:start + n]
        if out_expert_x_scale is not None and expected.scales[le] is not None:
            gs = out_expert_x_scale.cpu().to(torch.float32)[start:start + n]
            got = torch.cat([got, gs], dim=1)
            want = torch.cat([want, expected.scales[le]], dim=1)
        torch.testing.assert_close(_sort_rows(got), _sort_rows(want), rtol=0, atol=0,
                                   msg=lambda m, le=le: f"local expert {le}: {m}")


def expected_combine(
    x_times: torch.Tensor,
    weights: torch.Tensor,
    indices: torch.Tensor,
    num_experts: int,
    previous: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Combine output when every expert computes the same row-wise function ``f`` and
    ``x_times = f(x)`` is given per source token: ``sum_k w[t, k] * f(x[t])``."""
    w = weights.to(torch.float32).cpu().clone()
    w[indices.to(torch.int64).cpu() >= num_experts] = 0
    out = x_times.to(torch.float32).cpu() * w.sum(dim=1, keepdim=True)
    if previous is not None:
        out = out + previous.to(torch.float32).cpu()
    return out


def quantize_1x128(x: torch.Tensor, pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """float32 reference of block-scaled e4m3 quantisation: one scale per 128 contiguous
    elements, ``scale = max(amax, 1e-10) / 448`` (rounded up to a power of two with ``pow2``),
    values rounded to nearest-even and saturated. Returns (e4m3 tensor, float32 scales
    [tokens, hidden / 128])."""
    t, h = x.shape
    blocks = x.to(torch.float32).reshape(t, h // 128, 128)
    amax = blocks.abs().amax(dim=-1).clamp_min(1e-10)
    scale = amax * (1.0 / 448.0)
    if pow2:
        scale = ((scale.contiguous().view(torch.int32) + 0x007FFFFF) & 0x7F800000).view(torch.float32)
    q = (blocks * (1.0 / scale).unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(t, h), scale
