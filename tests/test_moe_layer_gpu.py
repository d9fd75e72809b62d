"""The fused MoE layer against a float32 PyTorch statement of the same layer (with the same
quantisation points), on one GPU and across GPUs."""

from __future__ import annotations

import pytest
import torch

from pplx_garden.distributed import ParallelLaunch
from pplx_garden.ops import dequantize_128x128, dequantize_1x128, quantize_1x128

pytestmark = pytest.mark.gpu


def _reference(x, indices, weights, w13_q, w13_s, w2_q, w2_s, experts_per_rank_offset=0):
    """out[t] = sum_k w[t,k] * FFN_{e(t,k)}(x[t]) with fp8 quantisation at the same places."""
    xq, xs = quantize_1x128(x.float().cpu())
    xd = dequantize_1x128(xq, xs)
    w13 = dequantize_128x128(w13_q.cpu(), w13_s.cpu())
    w2 = dequantize_128x128(w2_q.cpu(), w2_s.cpu())
    I = w2.shape[-1]
    out = torch.zeros_like(xd)
    idx = indices.cpu().to(torch.int64)
    for t in range(x.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            d = w13[e] @ xd[t]
            act = torch.nn.functional.silu(d[:I]) * d[I:]
            aq, a_s = quantize_1x128(act.unsqueeze(0))
            y = (w2[e] @ dequantize_1x128(aq, a_s)[0]).to(torch.bfloat16).float()
            out[t] += weights[t, k].item() * y
    return out


def test_single_gpu_layer_matches_reference() -> None:
    from pplx_garden.models import ExpertParallelMoE, route_topk

    dev = torch.device("cuda", 0)
    H, I, E, K, T = 512, 256, 8, 2, 48
    layer = ExpertParallelMoE(hidden_dim=H, intermediate_dim=I, num_experts=E, num_experts_per_token=K,
                              max_num_tokens=T, device=dev, global_group=None, init_std=0.05)
    try:
        gen = torch.Generator(device="cpu").manual_seed(3)
        x = torch.randn((T, H), generator=gen).to(torch.bfloat16).to(dev)
        indices, weights = route_topk(torch.randn((T, E), generator=gen).to(dev), K)
        out = layer(x, indices, weights)
        torch.cuda.synchronize()
        layer.check()
        want = _reference(x, indices.view(torch.int32), weights.cpu(), layer.w13, layer.w13_scale, layer.w2, layer.w2_scale)
        got = out.float().cpu()
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 1e-3, f"max abs error {err} vs scale {want.abs().max().item()}"
    finally:
        layer.destroy()


def _worker(device, dp_group, global_group, seed):
    from pplx_garden.models import ExpertParallelMoE, route_topk

    H, I, E, K, T = 512, 256, 16, 4, 64
    world, rank = global_group.size, global_group.rank
    L = E // world
    gen = torch.Generator(device="cpu").manual_seed(seed)
    w13_all = torch.randn((E, 2 * I, H), generator=gen) * 0.05
    w2_all = torch.randn((E, H, I), generator=gen) * 0.05
    layer = ExpertParallelMoE(hidden_dim=H, intermediate_dim=I, num_experts=E, num_experts_per_token=K,
                              max_num_tokens=T, device=device, global_group=global_group,
                              w13=w13_all[rank * L:(rank + 1) * L], w2=w2_all[rank * L:(rank + 1) * L])
    try:
        g2 = torch.Generator(device="cpu").manual_seed(seed + 1 + rank)
        x = torch.randn((T, H), generator=g2).to(torch.bfloat16).to(device)
        indices, weights = route_topk(torch.randn((T, E), generator=g2).to(device), K)
        out = layer(x, indices, weights)
        torch.cuda.synchronize()
        layer.check()
        from pplx_garden.ops import quantize_128x128

        w13_q, w13_s = quantize_128x128(w13_all)
        w2_q, w2_s = quantize_128x128(w2_all)
        want = _reference(x, indices.view(torch.int32), weights.cpu(), w13_q, w13_s, w2_q, w2_s)
        got = out.float().cpu()
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 1e-3, f"rank {rank}: max abs error {err}"
    finally:
        layer.destroy()
    return True


@pytest.mark.parametrize("world", [2, 4])
def test_multi_gpu_layer_matches_reference(world: int) -> None:
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    assert all(ParallelLaunch(world_size=world).run(_worker, 11))
