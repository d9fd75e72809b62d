"""The library-collective baseline against the oracle, as Gloo ranks on CPU."""

from __future__ import annotations

import pytest
import torch

from pplx_garden.distributed import ParallelLaunch
from pplx_garden.kernels import oracle
from tests.a2a_data import act, make_rank_data


def _worker(device, dp_group, global_group, cfg):
    from pplx_garden.kernels.nccl_all_to_all import NcclAllToAll

    world = global_group.size if global_group is not None else 1
    rank = global_group.rank if global_group is not None else 0
    tokens, experts, hidden, topk, padding, hscale = cfg
    a2a = NcclAllToAll(max_num_tokens=tokens, num_experts=experts, expert_padding=padding,
                       hidden_dim=hidden, hidden_dim_scale=hscale, in_dtype=torch.float32,
                       out_dtype=torch.float32, scale_dtype=torch.float32 if hscale else None,
                       num_experts_per_token=topk, device=device, global_group=global_group)
    data = [make_rank_data(seed=g, num_experts=experts, topk=topk, num_tokens=tokens,
                           hidden_dim=hidden, hidden_dim_scale=hscale, in_dtype=torch.float32,
                           device=device) for g in range(world)]
    mine = data[rank]
    L = oracle.experts_per_rank(experts, world)
    rows = tokens * world * min(topk, L) + L * padding
    for split in (False, True):
        num = torch.zeros(L, dtype=torch.int32)
        ox = torch.zeros((rows, hidden))
        osc = torch.zeros((rows, hscale)) if hscale else None
        out = torch.zeros((tokens, hidden))
        if split:
            a2a.dispatch(num, ox, osc, mine.dp_x, mine.dp_x_scale, mine.indices, mine.weights, do_recv=False)
            a2a.dispatch(num, ox, osc, mine.dp_x, mine.dp_x_scale, mine.indices, mine.weights, do_send=False)
        else:
            a2a.dispatch(num, ox, osc, mine.dp_x, mine.dp_x_scale, mine.indices, mine.weights)
        exp = oracle.expected_dispatch(rank, world, experts, padding, [d.dp_x for d in data],
                                       [d.dp_x_scale for d in data] if hscale else None,
                                       [d.indices for d in data])
        oracle.check_dispatch(exp, num, ox, osc)
        y = act(ox, osc)
        a2a.combine(out, mine.indices, mine.weights, y)
        torch.testing.assert_close(out, act(mine.dp_x, mine.dp_x_scale), rtol=1e-5, atol=1e-5)
    a2a.destroy()
    return True


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("cfg", [(16, 8, 32, 2, 1, None), (9, 12, 16, 3, 4, 2)])
def test_baseline_matches_oracle(world: int, cfg) -> None:
    assert all(ParallelLaunch(world_size=world).run(_worker, cfg))


def _layout_worker(device, dp_group, global_group, mismatch):
    """Every rank computes the all-to-all layout and compares it with its peers' (the check that
    P2PAllToAll makes before any rank writes into another's buffers)."""
    from pplx_garden.kernels.p2p_all_to_all import check_layout_agreement
    from pplx_garden.native.p2p_all_to_all import AllToAllContext

    rank, world = global_group.rank, global_group.size
    wire = "plain" if (mismatch and rank == 1) else "ll"
    layout = AllToAllContext.layout(hidden_dim=256, in_elemsize=2, out_elemsize=2, max_num_tokens=16,
                                    num_experts=8, num_experts_per_token=2, world_size=world, wire=wire,
                                    num_blocks=16 + rank)   # the launch shape may differ
    try:
        check_layout_agreement(global_group, rank, layout)
    except ValueError as e:
        return str(e)
    return "agreed"


def test_ranks_compare_their_all_to_all_layouts() -> None:
    assert ParallelLaunch(world_size=2).run(_layout_worker, False) == ["agreed", "agreed"]
    messages = ParallelLaunch(world_size=2).run(_layout_worker, True)
    assert all("disagree about the all-to-all layout" in m and "wire" in m for m in messages), messages
