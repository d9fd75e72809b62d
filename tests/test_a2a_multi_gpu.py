"""P2PAllToAll across real GPUs (one process per GPU, NVLink peer memory shared through
CUDA VMM file descriptors). Shapes follow the reference's table
(tests/p2p_all_to_all/test_p2p_all_to_all.py:240-557)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import pytest
import torch

from pplx_garden.distributed import ParallelLaunch
from pplx_garden.kernels import oracle
from tests.a2a_data import act, make_rank_data

pytestmark = pytest.mark.gpu


@dataclass
class Cfg:
    world: int
    dp_size: int = 1
    tokens: int = 128
    experts: int = 16
    hidden: int = 128
    hidden_scale: Optional[int] = None
    topk: int = 2
    in_dtype: torch.dtype = torch.float32
    out_dtype: torch.dtype = torch.float32
    padding: int = 1
    combine_mode: str = "per_route"
    iterations: int = 3


def _worker(device, dp_group, global_group, cfg: Cfg):
    from pplx_garden.kernels.p2p_all_to_all import P2PAllToAll

    rank, world = global_group.rank, global_group.size
    groups = world // cfg.dp_size
    my_group = rank // cfg.dp_size
    a2a = P2PAllToAll(
        max_num_tokens=cfg.tokens, num_experts=cfg.experts, expert_padding=cfg.padding,
        hidden_dim=cfg.hidden, hidden_dim_scale=cfg.hidden_scale, in_dtype=cfg.in_dtype,
        out_dtype=cfg.out_dtype, scale_dtype=torch.float32 if cfg.hidden_scale else None,
        num_experts_per_token=cfg.topk, nets_per_gpu=1, max_private_tokens=None, device=device,
        dp_group=dp_group if cfg.dp_size > 1 else None, node_group=None, global_group=global_group,
        combine_mode=cfg.combine_mode, wait_limit_ms=5000)
    try:
        L = a2a.num_local_experts
        rows = a2a.max_recv_rows
        for it in range(cfg.iterations):
            gen_dtype = torch.float32 if cfg.in_dtype == torch.float8_e4m3fn else cfg.in_dtype
            data = [make_rank_data(seed=1000 * it + g, num_experts=cfg.experts, topk=cfg.topk,
                                   num_tokens=cfg.tokens, hidden_dim=cfg.hidden,
                                   hidden_dim_scale=cfg.hidden_scale, in_dtype=gen_dtype,
                                   device=device) for g in range(groups)]
            if cfg.in_dtype == torch.float8_e4m3fn:
                for d in data:
                    d.dp_x = d.dp_x.clamp(-400, 400).to(torch.float8_e4m3fn)
            mine = data[my_group]
            num = torch.full((L,), -1, dtype=torch.int32, device=device)
            ox = torch.zeros((rows, cfg.hidden), dtype=torch.float32, device=device).to(cfg.in_dtype)
            osc = (torch.zeros((rows, cfg.hidden_scale), dtype=torch.float32, device=device)
                   if cfg.hidden_scale else None)
            out = torch.zeros((cfg.tokens, cfg.hidden), dtype=cfg.out_dtype, device=device)
            split = it % 2 == 1
            if split:
                a2a.dispatch(num, ox, osc, mine.dp_x, mine.dp_x_scale, mine.indices, mine.weights,
                             do_recv=False)
                a2a.dispatch(num, ox, osc, mine.dp_x, mine.dp_x_scale, mine.indices, mine.weights,
                             do_send=False)
            else:
                a2a.dispatch(num, ox, osc, mine.dp_x, mine.dp_x_scale, mine.indices, mine.weights)
            y = act(ox, osc).to(cfg.out_dtype)
            if split:
                a2a.combine(out, mine.indices, mine.weights, y, do_recv=False)
                a2a.combine(out, mine.indices, mine.weights, y, do_send=False)
            else:
                a2a.combine(out, mine.indices, mine.weights, y)
            torch.cuda.synchronize()
            a2a.check()
            exp = oracle.expected_dispatch(
                rank, world, cfg.experts, cfg.padding, [d.dp_x.cpu() for d in data],
                [d.dp_x_scale.cpu() for d in data] if cfg.hidden_scale else None,
                [d.indices.cpu() for d in data])
            oracle.check_dispatch(exp, num, ox, osc)
            want = act(mine.dp_x.cpu() if cfg.hidden_scale else mine.dp_x.cpu().to(torch.float32),
                       None if mine.dp_x_scale is None else mine.dp_x_scale.cpu())
            want = want.to(cfg.out_dtype).to(torch.float32)
            tol = dict(rtol=1e-5, atol=1e-5) if cfg.out_dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
            if cfg.hidden_scale:
                tol = dict(rtol=3e-2, atol=0.5)
            torch.testing.assert_close(out.cpu().to(torch.float32), want, **tol)
    finally:
        a2a.destroy()
    return True


CONFIGS = {
    "W2-FP32": Cfg(world=2),
    "W2-BF16-PADDED": Cfg(world=2, tokens=8, hidden=16, in_dtype=torch.bfloat16,
                          out_dtype=torch.bfloat16, padding=16),
    "W2-SCALES": Cfg(world=2, tokens=2, hidden_scale=16, in_dtype=torch.bfloat16,
                     out_dtype=torch.bfloat16),
    "W2-FP8-DEEPSEEK": Cfg(world=2, tokens=128, experts=256, hidden=7168, hidden_scale=56, topk=8,
                           in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16),
    "W2-PRE-REDUCE": Cfg(world=2, tokens=64, experts=32, hidden=1024, topk=4,
                         in_dtype=torch.bfloat16, out_dtype=torch.bfloat16, combine_mode="pre_reduce"),
    "W4-FP32-K8": Cfg(world=4, experts=128, topk=8),
    "W4-DP2-TINY": Cfg(world=4, dp_size=2, tokens=1, experts=4, hidden=8, topk=1,
                       in_dtype=torch.bfloat16, out_dtype=torch.bfloat16),
    "W4-BF16-H7168": Cfg(world=4, experts=256, hidden=7168, topk=8, in_dtype=torch.bfloat16,
                         out_dtype=torch.bfloat16),
    "W8-BF16": Cfg(world=8, experts=128, hidden=7168, topk=8, in_dtype=torch.bfloat16,
                   out_dtype=torch.bfloat16),
    "W8-FP8": Cfg(world=8, tokens=256, experts=128, hidden=7168, hidden_scale=56, topk=8,
                  in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16),
    "W8-DP2": Cfg(world=8, dp_size=2, tokens=32, experts=64, hidden=512, topk=4,
                  in_dtype=torch.bfloat16, out_dtype=torch.bfloat16),
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_p2p_all_to_all(name: str) -> None:
    cfg = CONFIGS[name]
    if torch.cuda.device_count() < cfg.world:
        pytest.skip(f"needs {cfg.world} GPUs")
    dp = cfg.dp_size if cfg.dp_size > 1 else None
    results = ParallelLaunch(world_size=cfg.world, dp_size=dp).run(_worker, cfg)
    assert all(results)
