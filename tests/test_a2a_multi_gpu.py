"""P2PAllToAll across real GPUs (one process per GPU, NVLink peer memory shared through
CUDA VMM file descriptors). Shapes follow the reference's table
(tests/p2p_all_to_all/test_p2p_all_to_all.py:240-557)."""

from __future__ import annotations

import contextlib
import os
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
    nvlink_group: Optional[int] = None   # ranks per "node"; None: all ranks share one NVLink domain


def _worker(device, dp_group, global_group, cfg: Cfg):
    from pplx_garden.kernels.p2p_all_to_all import P2PAllToAll

    rank, world = global_group.rank, global_group.size
    groups = world // cfg.dp_size
    my_group = rank // cfg.dp_size
    node_group = None
    if cfg.nvlink_group is not None:
        # slices the box into "nodes" of nvlink_group ranks: traffic between them goes through the
        # transfer engine and the host proxy (reference tests :304, :509-529)
        node_group = global_group.slice_by_count(world // cfg.nvlink_group)
    a2a = P2PAllToAll(
        max_num_tokens=cfg.tokens, num_experts=cfg.experts, expert_padding=cfg.padding,
        hidden_dim=cfg.hidden, hidden_dim_scale=cfg.hidden_scale, in_dtype=cfg.in_dtype,
        out_dtype=cfg.out_dtype, scale_dtype=torch.float32 if cfg.hidden_scale else None,
        num_experts_per_token=cfg.topk, nets_per_gpu=1, max_private_tokens=None, device=device,
        dp_group=dp_group if cfg.dp_size > 1 else None, node_group=node_group, global_group=global_group,
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


@contextlib.contextmanager
def _eager_module_loading(enable: bool):
    """With ranks served by the host proxy over the intra-box provider, the copies a running
    dispatch waits for are executed by this very GPU. CUDA's lazy module loading makes the first
    launch of any kernel (the test's own torch ops included) wait for the kernels that are
    running, and holds back copies meanwhile: the two would wait for each other until the bounded
    waits run out. The workers are fresh processes and inherit the setting."""
    old = os.environ.get("CUDA_MODULE_LOADING")
    if enable:
        os.environ["CUDA_MODULE_LOADING"] = "EAGER"
    try:
        yield
    finally:
        if enable:
            if old is None:
                os.environ.pop("CUDA_MODULE_LOADING", None)
            else:
                os.environ["CUDA_MODULE_LOADING"] = old


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
    "W2-NODES-OF-1": Cfg(world=2, tokens=32, experts=16, hidden=256, topk=4, in_dtype=torch.bfloat16,
                         out_dtype=torch.bfloat16, nvlink_group=1, iterations=4),
    "W2-NODES-OF-1-FP8-PRE": Cfg(world=2, tokens=64, experts=32, hidden=1024, hidden_scale=8, topk=4,
                                 in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16, nvlink_group=1,
                                 combine_mode="pre_reduce"),
    "W4-NODES-OF-2": Cfg(world=4, tokens=48, experts=32, hidden=512, topk=4, in_dtype=torch.bfloat16,
                         out_dtype=torch.bfloat16, padding=8, nvlink_group=2, iterations=4),
    "W4-NODES-OF-2-DP2": Cfg(world=4, dp_size=2, tokens=16, experts=16, hidden=256, topk=2,
                             in_dtype=torch.bfloat16, out_dtype=torch.bfloat16, nvlink_group=2),
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
    with _eager_module_loading(cfg.nvlink_group is not None):
        results = ParallelLaunch(world_size=cfg.world, dp_size=dp).run(_worker, cfg)
    assert all(results)


def _failing_worker(device, dp_group, global_group):
    """Two one-rank "nodes"; rank 0's engine fails its next write. The failure is made on the host,
    in the provider decorator; every device-side wait is bounded, so both ranks come back."""
    from pplx_garden.kernels.p2p_all_to_all import P2PAllToAll

    rank, world = global_group.rank, global_group.size
    node_group = global_group.slice_by_count(world)
    tokens, experts, hidden, topk = 16, 8, 128, 2
    a2a = P2PAllToAll(
        max_num_tokens=tokens, num_experts=experts, expert_padding=1, hidden_dim=hidden,
        hidden_dim_scale=None, in_dtype=torch.bfloat16, out_dtype=torch.bfloat16, scale_dtype=None,
        num_experts_per_token=topk, nets_per_gpu=1, max_private_tokens=None, device=device,
        dp_group=None, node_group=node_group, global_group=global_group, wait_limit_ms=1500)
    outcome = "no error"
    try:
        d = make_rank_data(seed=rank, num_experts=experts, topk=topk, num_tokens=tokens, hidden_dim=hidden,
                           hidden_dim_scale=None, in_dtype=torch.bfloat16, device=device)
        L, rows = a2a.num_local_experts, a2a.max_recv_rows
        num = torch.zeros(L, dtype=torch.int32, device=device)
        ox = torch.zeros((rows, hidden), dtype=torch.bfloat16, device=device)
        out = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device=device)
        # one clean layer first
        a2a.dispatch(num, ox, None, d.dp_x, None, d.indices, d.weights)
        a2a.combine(out, d.indices, d.weights, ox)
        torch.cuda.synchronize()
        a2a.check()
        global_group.barrier()
        if rank == 0:
            a2a._engine._inject_write_failure(device.index, 1)
        try:
            for _ in range(2):
                a2a.dispatch(num, ox, None, d.dp_x, None, d.indices, d.weights)
                a2a.combine(out, d.indices, d.weights, ox)
                torch.cuda.synchronize()
                a2a.check()
        except (RuntimeError, TimeoutError) as exc:
            outcome = str(exc)
        # the device is still usable
        assert torch.ones(4, device=device).sum().item() == 4
    finally:
        a2a.destroy()
    return outcome


def test_failed_transfer_surfaces_as_an_error_on_the_next_call() -> None:
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with _eager_module_loading(True):
        outcomes = ParallelLaunch(world_size=2).run(_failing_worker)
    assert "fabric-lib transfer error" in outcomes[0], outcomes     # the rank whose write failed
    assert outcomes[1] != "no error", outcomes                      # its peer ran into a bounded wait
